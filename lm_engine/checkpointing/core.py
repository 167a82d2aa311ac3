def ensure_last_checkpoint_is_saved():
    return None


def save_checkpoint(*args, **kwargs):
    raise NotImplementedError


def load_checkpoint_for_training(*args, **kwargs):
    raise NotImplementedError


def load_checkpoint_for_inference(*args, **kwargs):
    raise NotImplementedError


def save_args(*args, **kwargs):
    raise NotImplementedError
