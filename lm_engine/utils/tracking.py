"""Progress bar and experiment tracker front-ends (aim / wandb), resumable across restarts.

Parity: lm_engine/utils/tracking.py:26-183.
"""

from __future__ import annotations

import os
from typing import Any

from ..enums import ExperimentsTrackerName
from .packages import is_aim_available, is_wandb_available
from .parallel import is_tracking_rank, run_rank_n
from .pydantic import BaseArgs


class ProgressBar:
    """tqdm bar that only exists on global rank 0."""

    def __init__(self, start: int, end: int, desc: str | None = None) -> None:
        self.progress_bar = self._make(start, end, desc)

    @staticmethod
    @run_rank_n
    def _make(start: int, end: int, desc: str | None):
        from tqdm import trange

        return trange(start, end, desc=desc)

    def update(self, n: int = 1) -> None:
        if self.progress_bar is not None:
            self.progress_bar.update(n)

    def track(self, **metrics) -> None:
        if self.progress_bar is not None:
            self.progress_bar.set_postfix(**metrics)


class ExperimentsTracker:
    """Forwards scalars to aim or wandb from the tracking rank; a no-op everywhere else."""

    def __init__(
        self,
        experiments_tracker_name: ExperimentsTrackerName | None,
        aim_args: BaseArgs | None,
        wandb_args: BaseArgs | None,
        checkpoint_metadata: dict | None = None,
    ) -> None:
        self.tracker_name = experiments_tracker_name
        self.run = None
        self.wandb = None
        self.tracking_enabled = experiments_tracker_name is not None and is_tracking_rank()
        if not self.tracking_enabled:
            return

        job_id = os.environ.get("JOB_ID")
        if experiments_tracker_name == ExperimentsTrackerName.aim:
            if not is_aim_available():
                raise ImportError("aim is requested as experiments tracker but is not installed")
            from aim import Run

            run_hash = None if checkpoint_metadata is None else checkpoint_metadata.get("run_hash")
            self.run = Run(run_hash=run_hash, experiment=aim_args.experiment, repo=aim_args.repo)
            if job_id is not None:
                self.run["job_id"] = job_id
        elif experiments_tracker_name == ExperimentsTrackerName.wandb:
            if not is_wandb_available():
                raise ImportError("wandb is requested as experiments tracker but is not installed")
            import wandb

            self.wandb = wandb
            resume_id = None if checkpoint_metadata is None else checkpoint_metadata.get("id")
            self.run = wandb.init(
                project=wandb_args.project,
                name=wandb_args.name,
                entity=wandb_args.entity,
                id=resume_id,
                resume="must" if resume_id is not None else None,
            )
            # all curves share one x axis named "iteration"
            wandb.define_metric("iteration", hidden=True)
            wandb.define_metric("*", step_metric="iteration", step_sync=True)
        else:
            raise ValueError(f"unexpected experiments tracker ({experiments_tracker_name})")

    def log_args(self, args: BaseArgs) -> None:
        if not self.tracking_enabled:
            return
        flat = args.to_dict()
        if self.tracker_name == ExperimentsTrackerName.aim:
            self.run["args"] = flat
        else:
            self.run.config.update(flat, allow_val_change=True)

    def track(self, values: dict[str, Any], step: int | None = None, context: str | None = None) -> None:
        if not self.tracking_enabled:
            return
        if self.tracker_name == ExperimentsTrackerName.aim:
            ctx = None if context is None else {"subset": context}
            for key, value in values.items():
                self.run.track(value=value, name=key, step=step, context=ctx)
        else:
            prefix = "" if context is None else f"{context}-"
            payload = {f"{prefix}{k}": v for k, v in values.items()}
            payload["iteration"] = step
            self.wandb.log(payload)

    def finish(self) -> None:
        if not self.tracking_enabled:
            return
        if self.tracker_name == ExperimentsTrackerName.aim:
            self.run.close()
        else:
            self.run.finish()

    def state_dict(self) -> dict:
        if not self.tracking_enabled:
            return {}
        if self.tracker_name == ExperimentsTrackerName.aim:
            return {"run_hash": self.run.hash}
        return {"id": self.run.id}
