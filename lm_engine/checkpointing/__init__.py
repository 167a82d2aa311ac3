from .core import (
    ensure_last_checkpoint_is_saved,
    load_checkpoint_for_inference,
    load_checkpoint_for_training,
    save_args,
    save_checkpoint,
)
