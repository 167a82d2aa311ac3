"""``python -m lm_engine.unshard --config cfg.yml``: consolidate a training checkpoint into Hugging Face style
safetensors + config (+ tokenizer) under ``unsharded_path`` (parity: lm_engine/unshard.py:11-21)."""

from __future__ import annotations

from .arguments import UnshardingArgs, get_args
from .checkpointing import load_checkpoint_for_inference
from .enums import Mode
from .utils import ProcessGroupManager, run_rank_n


def main(argv: list[str] | None = None) -> None:
    args: UnshardingArgs = get_args(Mode.unsharding, argv)
    wrapper, _, state_dict = load_checkpoint_for_inference(args, Mode.unsharding, use_meta=True)
    run_rank_n(wrapper.save_pretrained, barrier=ProcessGroupManager.is_initialized())(args.unsharded_path, state_dict=state_dict)


if __name__ == "__main__":
    main()
