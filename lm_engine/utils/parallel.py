"""Process-group manager: one logical mesh ``(pp, ddp, fsdp, tp)`` with ``tp`` varying fastest, plus an expert
parallel view carved out of the data-parallel ranks.

Parity: lm_engine/utils/parallel.py:48-420 of the reference (same getter names, the ``set_dummy_*`` context
managers and ``run_rank_n``). Differences by design: the device type follows the machine (CPU ranks talk gloo, CUDA
ranks talk NCCL, so the plumbing runs without a GPU), the timeout really is in minutes, and an ``ep`` dimension
exists for expert parallelism.
"""

from __future__ import annotations

import os
from contextlib import contextmanager
from datetime import timedelta
from typing import Callable

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

from .miscellaneous import divide_if_divisible


class _State:
    mesh: DeviceMesh | None = None
    device_type: str = "cpu"
    global_rank: int | None = None
    local_rank: int | None = None
    world_size: int | None = None
    zero_stage: int = 3
    ep_world_size: int = 1
    ep_group: dist.ProcessGroup | None = None
    ep_rank: int | None = None
    dp_group: dist.ProcessGroup | None = None
    cpu_group: dist.ProcessGroup | None = None
    symmetric_memory_enabled: bool = False
    # overrides installed by the set_dummy_* context managers
    dummy: dict = {}


def _env_int(name: str, default: int) -> int:
    return int(os.environ.get(name, default))


class ProcessGroupManager:
    """Static accessor for ranks, sizes, meshes and groups of the current job."""

    def __init__(
        self,
        tensor_parallel_world_size: int = 1,
        pipeline_parallel_world_size: int = 1,
        data_parallel_replication_world_size: int | None = None,
        data_parallel_sharding_world_size: int | None = None,
        zero_stage: int = 3,
        timeout_minutes: int | None = None,
        use_async_tensor_parallel: bool = False,
        expert_parallel_world_size: int = 1,
        device_type: str | None = None,
    ) -> None:
        if device_type is None:
            device_type = "cuda" if torch.cuda.is_available() else "cpu"
        _State.device_type = device_type
        _State.zero_stage = zero_stage

        _State.global_rank = _env_int("RANK", 0)
        _State.local_rank = _env_int("LOCAL_RANK", 0)
        _State.world_size = _env_int("WORLD_SIZE", 1)

        if device_type == "cuda":
            torch.cuda.set_device(_State.local_rank)

        if not dist.is_initialized():
            kwargs = {}
            if timeout_minutes is not None:
                kwargs["timeout"] = timedelta(minutes=timeout_minutes)
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            backend = "cpu:gloo,cuda:nccl" if device_type == "cuda" else "gloo"
            dist.init_process_group(backend=backend, rank=_State.global_rank, world_size=_State.world_size, **kwargs)

        world = _State.world_size
        tp, pp = tensor_parallel_world_size, pipeline_parallel_world_size
        dp = divide_if_divisible(world, tp * pp, "world size must be divisible by tp * pp")

        rep, shard = data_parallel_replication_world_size, data_parallel_sharding_world_size
        if zero_stage == 0:
            assert rep in (None, dp) and shard in (None, 1), "ZeRO stage 0 replicates over all data parallel ranks"
            rep, shard = dp, 1
        elif rep is None and shard is None:
            rep, shard = 1, dp
        elif rep is None:
            rep = divide_if_divisible(dp, shard, "")
        elif shard is None:
            shard = divide_if_divisible(dp, rep, "")
        assert rep * shard == dp, "replication x sharding must equal the data parallel world size"

        _State.mesh = init_device_mesh(device_type, (pp, rep, shard, tp), mesh_dim_names=("pp", "ddp", "fsdp", "tp"))
        _State.dp_group = None
        _State.cpu_group = None

        # expert parallel groups: consecutive data-parallel ranks (same pp and tp coordinates)
        _State.ep_world_size = expert_parallel_world_size
        _State.ep_group = None
        _State.ep_rank = None
        if expert_parallel_world_size > 1:
            divide_if_divisible(dp, expert_parallel_world_size, "ep must divide the data parallel world size")
            dp_rank = ProcessGroupManager.get_data_parallel_rank()
            ranks_of_dp = ProcessGroupManager._ranks_along_dp()
            for start in range(0, dp, expert_parallel_world_size):
                members = ranks_of_dp[start : start + expert_parallel_world_size]
                # every rank must create every group, in the same order
                for pp_i in range(pp):
                    for tp_i in range(tp):
                        grp_ranks = [ProcessGroupManager._global_rank_of(pp_i, m, tp_i) for m in range(start, start + expert_parallel_world_size)]
                        grp = dist.new_group(grp_ranks)
                        if _State.global_rank in grp_ranks:
                            _State.ep_group = grp
                            _State.ep_rank = grp_ranks.index(_State.global_rank)
                del members
            assert _State.ep_group is not None and dp_rank is not None

        # asynchronous tensor parallelism = the sequence-parallel linears run their collective inside the GEMM kernel
        _State.symmetric_memory_enabled = bool(use_async_tensor_parallel and device_type == "cuda")

    @staticmethod
    def is_async_tensor_parallel_enabled() -> bool:
        return _State.symmetric_memory_enabled or os.environ.get("LM_ENGINE_FUSED_TP", "0") == "1"

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _global_rank_of(pp_i: int, dp_i: int, tp_i: int) -> int:
        tp = ProcessGroupManager.get_tensor_parallel_world_size()
        dp = ProcessGroupManager.get_data_parallel_world_size()
        return (pp_i * dp + dp_i) * tp + tp_i

    @staticmethod
    def _ranks_along_dp() -> list[int]:
        pp_i = ProcessGroupManager.get_pipeline_parallel_rank()
        tp_i = ProcessGroupManager.get_tensor_parallel_rank()
        dp = ProcessGroupManager.get_data_parallel_world_size()
        return [ProcessGroupManager._global_rank_of(pp_i, d, tp_i) for d in range(dp)]

    @staticmethod
    def is_initialized() -> bool:
        return dist.is_initialized() and _State.mesh is not None

    @staticmethod
    def get_device_type() -> str:
        return _State.device_type

    @staticmethod
    def get_device() -> torch.device:
        if _State.device_type == "cuda":
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    @staticmethod
    def get_mesh() -> DeviceMesh:
        return _State.mesh

    @staticmethod
    def get_zero_stage() -> int:
        return _State.zero_stage

    @staticmethod
    def get_global_rank() -> int:
        if _State.global_rank is None:
            return _env_int("RANK", 0)
        return _State.global_rank

    @staticmethod
    def get_local_rank() -> int:
        if _State.local_rank is None:
            return _env_int("LOCAL_RANK", 0)
        return _State.local_rank

    @staticmethod
    def get_world_size() -> int:
        if _State.world_size is None:
            return _env_int("WORLD_SIZE", 1)
        return _State.world_size

    # ------------------------------------------------------------------ tensor parallel
    @staticmethod
    def get_tensor_parallel_mesh() -> DeviceMesh:
        return _State.mesh["tp"]

    @staticmethod
    def get_tensor_parallel_group() -> dist.ProcessGroup:
        return _State.mesh["tp"].get_group()

    @staticmethod
    def get_tensor_parallel_rank() -> int:
        if "tp_rank" in _State.dummy:
            return _State.dummy["tp_rank"]
        if _State.mesh is None:
            return 0
        return _State.mesh["tp"].get_local_rank()

    @staticmethod
    def get_tensor_parallel_world_size() -> int:
        if "tp_world_size" in _State.dummy:
            return _State.dummy["tp_world_size"]
        if _State.mesh is None:
            return 1
        return _State.mesh["tp"].size()

    @staticmethod
    def is_tensor_parallel_enabled() -> bool:
        return ProcessGroupManager.get_tensor_parallel_world_size() > 1

    @staticmethod
    def is_tensor_parallel_first_rank() -> bool:
        return ProcessGroupManager.get_tensor_parallel_rank() == 0

    @staticmethod
    def get_tensor_parallel_first_rank() -> int:
        """Global rank of the member with tp-rank 0 in this rank's tensor parallel group."""
        if "tp_first_rank" in _State.dummy:
            return _State.dummy["tp_first_rank"]
        return dist.get_process_group_ranks(ProcessGroupManager.get_tensor_parallel_group())[0]

    @staticmethod
    @contextmanager
    def set_dummy_tensor_parallel_first_rank(rank: int):
        previous = _State.dummy.get("tp_first_rank")
        _State.dummy["tp_first_rank"] = rank
        try:
            yield
        finally:
            if previous is None:
                _State.dummy.pop("tp_first_rank", None)
            else:
                _State.dummy["tp_first_rank"] = previous

    @staticmethod
    @contextmanager
    def set_dummy_tensor_parallel_rank(rank: int):
        previous = _State.dummy.get("tp_rank")
        _State.dummy["tp_rank"] = rank
        try:
            yield
        finally:
            if previous is None:
                _State.dummy.pop("tp_rank", None)
            else:
                _State.dummy["tp_rank"] = previous

    @staticmethod
    @contextmanager
    def set_dummy_tensor_parallel_world_size(world_size: int):
        previous = _State.dummy.get("tp_world_size")
        _State.dummy["tp_world_size"] = world_size
        try:
            yield
        finally:
            if previous is None:
                _State.dummy.pop("tp_world_size", None)
            else:
                _State.dummy["tp_world_size"] = previous

    # ------------------------------------------------------------------ pipeline parallel
    @staticmethod
    def get_pipeline_parallel_mesh() -> DeviceMesh:
        return _State.mesh["pp"]

    @staticmethod
    def get_pipeline_parallel_group() -> dist.ProcessGroup:
        return _State.mesh["pp"].get_group()

    @staticmethod
    def get_pipeline_parallel_rank() -> int:
        if "pp_rank" in _State.dummy:
            return _State.dummy["pp_rank"]
        if _State.mesh is None:
            return 0
        return _State.mesh["pp"].get_local_rank()

    @staticmethod
    def get_pipeline_parallel_world_size() -> int:
        if "pp_world_size" in _State.dummy:
            return _State.dummy["pp_world_size"]
        if _State.mesh is None:
            return 1
        return _State.mesh["pp"].size()

    @staticmethod
    @contextmanager
    def set_dummy_pipeline_parallel_rank(rank: int):
        previous = _State.dummy.get("pp_rank")
        _State.dummy["pp_rank"] = rank
        try:
            yield
        finally:
            if previous is None:
                _State.dummy.pop("pp_rank", None)
            else:
                _State.dummy["pp_rank"] = previous

    @staticmethod
    @contextmanager
    def set_dummy_pipeline_parallel_world_size(world_size: int):
        previous = _State.dummy.get("pp_world_size")
        _State.dummy["pp_world_size"] = world_size
        try:
            yield
        finally:
            if previous is None:
                _State.dummy.pop("pp_world_size", None)
            else:
                _State.dummy["pp_world_size"] = previous

    # ------------------------------------------------------------------ data parallel
    @staticmethod
    def get_data_parallel_mesh() -> DeviceMesh:
        """2-D ``(ddp, fsdp)`` mesh: gradients are reduce-scattered over ``fsdp`` and all-reduced over ``ddp``."""
        return _State.mesh["ddp", "fsdp"]

    @staticmethod
    def get_replication_group() -> dist.ProcessGroup:
        return _State.mesh["ddp"].get_group()

    @staticmethod
    def get_sharding_group() -> dist.ProcessGroup:
        return _State.mesh["fsdp"].get_group()

    @staticmethod
    def get_replication_world_size() -> int:
        return 1 if _State.mesh is None else _State.mesh["ddp"].size()

    @staticmethod
    def get_sharding_world_size() -> int:
        return 1 if _State.mesh is None else _State.mesh["fsdp"].size()

    @staticmethod
    def get_data_parallel_replication_world_size() -> int:
        """The reference's name for :meth:`get_replication_world_size`."""
        return ProcessGroupManager.get_replication_world_size()

    @staticmethod
    def get_data_parallel_sharding_world_size() -> int:
        """The reference's name for :meth:`get_sharding_world_size`."""
        return ProcessGroupManager.get_sharding_world_size()

    @staticmethod
    def get_sharding_rank() -> int:
        return 0 if _State.mesh is None else _State.mesh["fsdp"].get_local_rank()

    @staticmethod
    def get_data_parallel_group() -> dist.ProcessGroup:
        if _State.dp_group is None:
            if _State.mesh["ddp"].size() == 1:
                _State.dp_group = _State.mesh["fsdp"].get_group()
            elif _State.mesh["fsdp"].size() == 1:
                _State.dp_group = _State.mesh["ddp"].get_group()
            else:
                _State.dp_group = _State.mesh["ddp", "fsdp"]._flatten("dp").get_group()
        return _State.dp_group

    @staticmethod
    def get_data_parallel_rank() -> int:
        if "dp_rank" in _State.dummy:
            return _State.dummy["dp_rank"]
        if _State.mesh is None:
            return 0
        return _State.mesh["ddp"].get_local_rank() * _State.mesh["fsdp"].size() + _State.mesh["fsdp"].get_local_rank()

    @staticmethod
    def get_data_parallel_world_size() -> int:
        if "dp_world_size" in _State.dummy:
            return _State.dummy["dp_world_size"]
        if _State.mesh is None:
            return 1
        return _State.mesh["ddp"].size() * _State.mesh["fsdp"].size()

    @staticmethod
    @contextmanager
    def set_dummy_data_parallel_rank(rank: int):
        previous = _State.dummy.get("dp_rank")
        _State.dummy["dp_rank"] = rank
        try:
            yield
        finally:
            if previous is None:
                _State.dummy.pop("dp_rank", None)
            else:
                _State.dummy["dp_rank"] = previous

    @staticmethod
    @contextmanager
    def set_dummy_data_parallel_world_size(world_size: int):
        previous = _State.dummy.get("dp_world_size")
        _State.dummy["dp_world_size"] = world_size
        try:
            yield
        finally:
            if previous is None:
                _State.dummy.pop("dp_world_size", None)
            else:
                _State.dummy["dp_world_size"] = previous

    # ------------------------------------------------------------------ expert parallel
    @staticmethod
    def get_expert_parallel_world_size() -> int:
        return _State.ep_world_size

    @staticmethod
    def get_expert_parallel_rank() -> int:
        return 0 if _State.ep_rank is None else _State.ep_rank

    @staticmethod
    def get_expert_parallel_group() -> dist.ProcessGroup | None:
        return _State.ep_group

    # ------------------------------------------------------------------ misc
    @staticmethod
    def get_cpu_group() -> dist.ProcessGroup | None:
        """A gloo group over all ranks for host-side object exchange (None when the default group is gloo)."""
        if _State.device_type == "cpu":
            return None
        if _State.cpu_group is None:
            _State.cpu_group = dist.new_group(backend="gloo")
        return _State.cpu_group

    @staticmethod
    def __str__() -> str:
        return str(_State.mesh)

    @staticmethod
    def destroy_process_groups() -> None:
        if dist.is_initialized():
            try:
                dist.barrier()
            finally:
                dist.destroy_process_group()
        _State.mesh = None
        _State.dp_group = None
        _State.cpu_group = None
        _State.ep_group = None


def run_rank_n(func: Callable, rank: int = 0, barrier: bool = False) -> Callable:
    """Wrap ``func`` so that only global rank ``rank`` executes it (others return None)."""

    def wrapped(*args, **kwargs):
        output = None
        if ProcessGroupManager.get_global_rank() == rank:
            output = func(*args, **kwargs)
        if barrier and dist.is_initialized():
            dist.barrier()
        return output

    return wrapped


def is_tracking_rank() -> bool:
    """The rank that logs metrics: first data-parallel and tensor-parallel rank of the LAST pipeline stage."""
    return (
        ProcessGroupManager.get_data_parallel_rank() == 0
        and ProcessGroupManager.is_tensor_parallel_first_rank()
        and ProcessGroupManager.get_pipeline_parallel_rank() == ProcessGroupManager.get_pipeline_parallel_world_size() - 1
    )


def get_pipeline_stage_ids_on_current_rank(num_pipeline_stages: int) -> tuple[int, ...]:
    """Interleaved assignment: rank r owns stages r, r + pp, r + 2 pp, ..."""
    pp_world = ProcessGroupManager.get_pipeline_parallel_world_size()
    per_rank = divide_if_divisible(num_pipeline_stages, pp_world, "number of stages must be a multiple of pp size")
    rank = ProcessGroupManager.get_pipeline_parallel_rank()
    return tuple(rank + i * pp_world for i in range(per_rank))
