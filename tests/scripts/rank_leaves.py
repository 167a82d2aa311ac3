"""Two or more CPU ranks (gloo): all of them finish one collective, then the last rank leaves between steps without a
word. The others must get an exception out of their next collective within the process-group timeout, not hang."""

import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from lm_engine.utils import ProcessGroupManager


def main() -> None:
    ProcessGroupManager(timeout_minutes=0.1)  # six seconds
    rank, world = dist.get_rank(), dist.get_world_size()
    value = torch.ones(4)
    dist.all_reduce(value)
    assert float(value[0]) == world
    if rank == world - 1:
        os._exit(0)  # between steps, nothing of this rank in flight
    started = time.monotonic()
    try:
        dist.all_reduce(value)
    except Exception as error:  # noqa: BLE001 - the point is that SOMETHING is raised
        print(f"rank {rank}: collective failed after {time.monotonic() - started:.1f} s: {type(error).__name__}", flush=True)
        os._exit(17)
    print(f"rank {rank}: the collective returned although a rank had left", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
