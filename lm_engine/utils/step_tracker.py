from __future__ import annotations


class StepTracker:
    """Batch-size bookkeeping shared by the drivers (parity: lm_engine/utils/step_tracker.py:12-29)."""

    _micro_batch_size: int | None = None
    _gradient_accumulation_steps: int | None = None

    def __init__(self, micro_batch_size: int, gradient_accumulation_steps: int) -> None:
        StepTracker._micro_batch_size = micro_batch_size
        StepTracker._gradient_accumulation_steps = gradient_accumulation_steps

    @staticmethod
    def get_micro_batch_size() -> int:
        return StepTracker._micro_batch_size

    @staticmethod
    def get_gradient_accumulation_steps() -> int:
        return StepTracker._gradient_accumulation_steps

    @staticmethod
    def get_local_batch_size() -> int:
        return StepTracker._micro_batch_size * StepTracker._gradient_accumulation_steps

    @staticmethod
    def get_global_batch_size() -> int:
        from .parallel import ProcessGroupManager

        return StepTracker.get_local_batch_size() * ProcessGroupManager.get_data_parallel_world_size()
