from .optimizer import FusedAdamW, build_optimizer, get_optimizer_container
from .params_group import get_param_groups_with_names
from .scheduler import PhasedSchedule, build_lr_scheduler, get_scheduler_container


def get_learning_rate(model_container, lr_scheduler) -> float:
    """Current learning rate of the first parameter group (parity: lm_engine/optimization/__init__.py:10-19)."""
    if lr_scheduler is None or (hasattr(lr_scheduler, "__len__") and len(lr_scheduler) and lr_scheduler[0] is None):
        for model in model_container:
            for param in model.parameters():
                return param._lr_scheduler.get_last_lr()[0]
    return lr_scheduler[0].get_last_lr()[0]
