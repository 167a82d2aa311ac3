"""Training checkpoints in the directory layout of the reference (lm_engine/checkpointing/__init__.py:43-398):

    save_path/latest_checkpointed_iteration.json
    save_path/global_step{N}/model/              torch.distributed.checkpoint, key "state" -> {parameter name: tensor}
    save_path/global_step{N}/optimizer/          same, flattened optimizer state ("state.<name>.exp_avg", ...)
    save_path/global_step{N}/model_optimizer/    both in one store when async_checkpointing is on
    save_path/global_step{N}/lr_scheduler/lr_scheduler-{rank}.pt
    save_path/global_step{N}/rng_state/rng_state-{rank}.pt
    save_path/global_step{N}/dataloader/dataloader-{dp_rank}.pt      (finetuning)
    save_path/global_step{N}/experiments_tracker.json, metadata.json, training_config.yml

The sharded engine stores parameters as flat slices, so for the distributed-checkpoint files every parameter (and its
optimizer moments) is re-expressed as a DTensor sharded on dim 0 over the ``fsdp`` mesh, which is the on-disk form of
the reference and lets checkpoints be reloaded on a different number of ranks. A file named ``KILLSWITCH`` in
``save_path`` makes the job exit cleanly after the next save. A checkpoint is written under
``global_step{N}.incomplete`` and renamed to ``global_step{N}`` once every shard is on disk; only then is
``latest_checkpointed_iteration.json`` replaced (atomically), so neither the directory nor the pointer ever names a
partial checkpoint.
"""

from __future__ import annotations

import json
import logging
import os
import random
import shutil
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
import yaml

from ..enums import Mode
from ..utils import ExperimentsTracker, ProcessGroupManager, load_yaml, log_rank_0, run_rank_n, string_to_torch_dtype

_KILLSWITCH = "KILLSWITCH"
_PENDING = None  # future of an in-flight asynchronous save


# ----------------------------------------------------------------------------------------------------------------------
# paths
def _base(path: str, iteration: int) -> str:
    return os.path.join(path, f"global_step{iteration}")


def _model_path(p): return os.path.join(p, "model")
def _optimizer_path(p): return os.path.join(p, "optimizer")
def _model_optimizer_path(p): return os.path.join(p, "model_optimizer")
def _lr_scheduler_path(p): return os.path.join(p, "lr_scheduler", f"lr_scheduler-{ProcessGroupManager.get_global_rank()}.pt")
def _rng_path(p): return os.path.join(p, "rng_state", f"rng_state-{ProcessGroupManager.get_global_rank()}.pt")
def _dataloader_path(p): return os.path.join(p, "dataloader", f"dataloader-{ProcessGroupManager.get_data_parallel_rank()}.pt")
def _tracker_path(p): return os.path.join(p, "experiments_tracker.json")
def _metadata_path(p): return os.path.join(p, "metadata.json")
def _latest_path(path): return os.path.join(path, "latest_checkpointed_iteration.json")
def _training_config_path(p): return os.path.join(p, "training_config.yml")


def _distributed() -> bool:
    return dist.is_initialized() and dist.get_world_size() > 1


def _barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


# ----------------------------------------------------------------------------------------------------------------------
# parameter <-> DTensor views
def _dim0_chunk(full: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The rank's piece under torch.chunk semantics (what ``Shard(0)`` means), possibly empty."""
    if full.dim() == 0:
        return full.clone() if rank == 0 else full.new_empty((0,))
    size = full.shape[0]
    per = -(-size // world)
    lo, hi = min(rank * per, size), min((rank + 1) * per, size)
    return full[lo:hi].clone()


def _as_sharded(full: torch.Tensor, engine) -> torch.Tensor:
    """Express a replicated full tensor as a DTensor sharded on dim 0 over the fsdp mesh (plain tensor on 1 rank)."""
    if not _distributed() or engine.shard_world == 1 and engine.replica_world == 1:
        return full
    from torch.distributed.tensor import DTensor, Replicate, Shard

    if full.dim() == 0:
        full = full.reshape(1)
    mesh = ProcessGroupManager.get_mesh()["fsdp"] if engine.replica_world == 1 else ProcessGroupManager.get_data_parallel_mesh()
    placements = [Shard(0)] if engine.replica_world == 1 else [Replicate(), Shard(0)]
    local = _dim0_chunk(full, engine.shard_world, engine.shard_rank)
    return DTensor.from_local(local, mesh, placements, run_check=False, shape=full.shape, stride=full.contiguous().stride())


def _to_full(value: torch.Tensor) -> torch.Tensor:
    if hasattr(value, "full_tensor"):
        return value.full_tensor()
    return value


def _as_expert_sharded(local: torch.Tensor, engine) -> torch.Tensor:
    """Expert-parallel parameters: every rank of the sharding group holds other experts, i.e. its tensor IS the rank's
    dim-0 shard of the bank of all experts."""
    if not _distributed() or engine.shard_world == 1:
        return local
    from torch.distributed.tensor import DTensor, Shard

    assert engine.replica_world == 1, "expert parallelism spans the sharding group of the engine"
    mesh = ProcessGroupManager.get_mesh()["fsdp"]
    shape = (local.shape[0] * engine.shard_world, *local.shape[1:])
    stride = torch.empty(shape, device="meta").stride()
    return DTensor.from_local(local.contiguous(), mesh, [Shard(0)], run_check=False, shape=torch.Size(shape), stride=stride)


def _tp_world() -> int:
    return ProcessGroupManager.get_tensor_parallel_world_size() if ProcessGroupManager.is_initialized() else 1


def _as_tp_sharded(local: torch.Tensor, dim: int, engine) -> torch.Tensor:
    """A tensor-parallel parameter: every tensor-parallel rank holds another block along ``dim``. On disk it is ONE
    tensor of the full shape, the ranks' blocks concatenated along ``dim`` in rank order (what a ``Shard(dim)`` DTensor
    over the ``tp`` mesh dimension means, and the form the reference writes; ``fix_unsharded_state_dict`` turns it into
    the single-device layout for gated and fused projections). Over the data-parallel dimensions the block is sharded
    on dim 0 when that is a different dimension, else replicated (one data-parallel rank writes it)."""
    from torch.distributed.tensor import DTensor, Replicate, Shard

    tp = _tp_world()
    local = local.contiguous()
    shape = list(local.shape)
    shape[dim] *= tp
    stride = torch.empty(shape, device="meta").stride()
    names, placements = [], []
    if engine.replica_world > 1:
        names.append("ddp")
        placements.append(Replicate())
    if engine.shard_world > 1:
        names.append("fsdp")
        if dim != 0 and local.shape[0] >= engine.shard_world:
            placements.append(Shard(0))
            local = _dim0_chunk(local, engine.shard_world, engine.shard_rank)
        else:
            placements.append(Replicate())
    names.append("tp")
    placements.append(Shard(dim))
    mesh = ProcessGroupManager.get_mesh()[tuple(names)] if len(names) > 1 else ProcessGroupManager.get_mesh()["tp"]
    return DTensor.from_local(local, mesh, placements, run_check=False, shape=torch.Size(shape), stride=stride)


def _view(unit, slot, full_slot: torch.Tensor, engine) -> torch.Tensor:
    if getattr(unit, "local_only", False):
        return _as_expert_sharded(full_slot, engine)
    dim = getattr(slot.param, "_tp_shard_dim", None)
    if dim is not None and _tp_world() > 1 and _distributed():
        return _as_tp_sharded(full_slot, dim % max(full_slot.dim(), 1), engine)
    return _as_sharded(full_slot, engine)


def _local_value(unit, value: torch.Tensor, engine) -> torch.Tensor:
    """What this rank keeps of a loaded tensor: everything, its own experts (expert-parallel units), or its own
    tensor-parallel block (a DTensor sharded over ``tp`` is gathered over the data-parallel dimensions only)."""
    if isinstance(value, torch.Tensor) and hasattr(value, "placements") and "tp" in (value.device_mesh.mesh_dim_names or ()):
        from torch.distributed.tensor import Replicate

        names = value.device_mesh.mesh_dim_names
        target = [p if n == "tp" else Replicate() for n, p in zip(names, value.placements)]
        return value.redistribute(value.device_mesh, target).to_local()
    full = _to_full(value) if isinstance(value, torch.Tensor) else value
    if getattr(unit, "local_only", False) and engine.shard_world > 1 and full.dim() > 0:
        return full.chunk(engine.shard_world, dim=0)[engine.shard_rank]
    return full


def _unit_full_fp32(unit, engine, source: str, optimizer=None) -> torch.Tensor:
    """Gather one flat quantity of a unit (``master``, ``exp_avg`` or ``exp_avg_sq``) from all shards."""
    from ..parallel.collectives import all_gather_in_place

    full = torch.zeros(unit.numel, dtype=torch.float32, device=unit.device)
    lo, hi = unit.shard_range
    if source == "master":
        full[lo:hi].copy_(unit.master)
    else:
        for seg in unit.segments:
            state = optimizer.state.get(seg.master, {})
            if source in state:
                full[lo + seg.start : lo + seg.start + seg.numel].copy_(state[source])
    if unit.world > 1:
        all_gather_in_place(full, unit.shard_numel, unit.rank, engine.shard_group)
    return full


def _scatter_unit_quantity(unit, full: torch.Tensor, source: str, optimizer) -> None:
    lo, _ = unit.shard_range
    for seg in unit.segments:
        state = optimizer.state.setdefault(seg.master, {})
        piece = full[lo + seg.start : lo + seg.start + seg.numel].to(seg.master.device)  # the host under cpu_offload
        if source not in state:
            state[source] = piece.clone()
        else:
            state[source].copy_(piece)


def get_model_state_dict(model_container) -> dict[str, torch.Tensor]:
    """``{name: fp32 tensor}`` over all local pipeline stages; names carry the wrapper prefix ``model.``."""
    out = {}
    for model in model_container:
        engine = getattr(model, "_lm_engine", None)
        if engine is None:
            out.update({k: v for k, v in model.state_dict().items() if not k.startswith("teacher_model.")})
            continue
        for unit in engine.units:
            full = _unit_full_fp32(unit, engine, "master")
            for slot in unit.slots:
                out[slot.name] = _view(unit, slot, full[slot.offset : slot.offset + slot.numel].view(slot.shape).clone(), engine)
            del full
    return out


def set_model_state_dict(model_container, state: dict[str, torch.Tensor]) -> None:
    for model in model_container:
        engine = getattr(model, "_lm_engine", None)
        if engine is None:
            model.load_state_dict({k: _to_full(v) for k, v in state.items()}, strict=False)
            continue
        for unit, slot in engine.named_slots():
            if slot.name in state:
                unit.adopt(slot, _local_value(unit, state[slot.name], engine).reshape(slot.shape).to(device=engine.device, dtype=torch.float32))


def _hyperparameters(group: dict) -> dict:
    return {k: v for k, v in group.items() if k not in ("params", "name")}


def get_optimizer_state_dict(model_container, optimizer_container) -> dict[str, object]:
    """Flattened optimizer state keyed by parameter name: ``state.<name>.<field>`` and ``param_groups.<name>.<key>``."""
    out: dict[str, object] = {}
    for model, optimizer in zip(model_container, optimizer_container):
        if optimizer is None:
            continue
        engine = getattr(model, "_lm_engine", None)
        if engine is None:
            names = {id(p): n for n, p in model.named_parameters()}
            for group in optimizer.param_groups:
                for p in group["params"]:
                    name = names[id(p)]
                    for field, value in optimizer.state.get(p, {}).items():
                        out[f"state.{name}.{field}"] = value
                    for key, value in _hyperparameters(group).items():
                        out[f"param_groups.{name}.{key}"] = value
            continue
        group_of_segment = {id(p): g for g in optimizer.param_groups for p in g["params"]}
        hyper_of_group_name: dict[str, dict] = {}
        step_of_group_name: dict[str, int] = {}
        for unit in engine.units:
            for seg in unit.segments:
                group = group_of_segment.get(id(seg.master))
                if group is not None:
                    hyper_of_group_name[seg.group] = _hyperparameters(group)
                    step = optimizer.state.get(seg.master, {}).get("step", 0)
                    step_of_group_name[seg.group] = int(step.item()) if isinstance(step, torch.Tensor) else int(step)
        for unit in engine.units:
            fields = sorted({f for seg in unit.segments for f, v in optimizer.state.get(seg.master, {}).items()
                             if isinstance(v, torch.Tensor) and v.dim() > 0 and v.numel() == seg.numel})
            fulls = {f: _unit_full_fp32(unit, engine, f, optimizer) for f in fields}
            for slot in unit.slots:
                for f, full in fulls.items():
                    out[f"state.{slot.name}.{f}"] = _view(unit, slot, full[slot.offset : slot.offset + slot.numel].view(slot.shape).clone(), engine)
                out[f"state.{slot.name}.step"] = torch.tensor(float(step_of_group_name.get(slot.group, 0)))
                for key, value in hyper_of_group_name.get(slot.group, {}).items():
                    out[f"param_groups.{slot.name}.{key}"] = value
            del fulls
    return out


def set_optimizer_state_dict(model_container, optimizer_container, state: dict[str, object]) -> None:
    for model, optimizer in zip(model_container, optimizer_container):
        if optimizer is None:
            continue
        engine = getattr(model, "_lm_engine", None)
        if engine is None:
            names = {n: p for n, p in model.named_parameters()}
            for key, value in state.items():
                kind, rest = key.split(".", 1)
                name, field = rest.rsplit(".", 1)
                if kind == "state" and name in names:
                    optimizer.state.setdefault(names[name], {})[field] = _to_full(value) if isinstance(value, torch.Tensor) else value
            continue
        for unit in engine.units:
            fields = sorted({key.rsplit(".", 1)[1] for key in state if key.startswith("state.") and
                             key.rsplit(".", 1)[0][len("state."):] in {s.name for s in unit.slots}} - {"step"})
            for f in fields:
                full = torch.zeros(unit.numel, dtype=torch.float32, device=unit.device)
                for slot in unit.slots:
                    key = f"state.{slot.name}.{f}"
                    if key in state:
                        full[slot.offset : slot.offset + slot.numel].copy_(_local_value(unit, state[key], engine).reshape(-1))
                _scatter_unit_quantity(unit, full, f, optimizer)
            for seg in unit.segments:
                first = next(s for s in unit.slots if s.group == seg.group)
                step = state.get(f"state.{first.name}.step")
                if step is not None:
                    optimizer.state.setdefault(seg.master, {})["step"] = int(float(_to_full(step))) if isinstance(step, torch.Tensor) else int(step)
        slot_of_group = {}
        for unit in engine.units:
            for slot in unit.slots:
                slot_of_group.setdefault(slot.group, slot.name)
        for group in optimizer.param_groups:
            name = slot_of_group.get(group.get("name"))
            if name is None:
                continue
            for key in list(_hyperparameters(group)):
                saved = state.get(f"param_groups.{name}.{key}")
                if saved is not None:
                    group[key] = saved


def _placeholders(reference_state: dict[str, object]) -> dict[str, object]:
    """Same keys / shapes / shardings as ``reference_state`` with zeroed storage, to be filled by ``dcp.load``."""
    out = {}
    for key, value in reference_state.items():
        if isinstance(value, torch.Tensor):
            out[key] = torch.zeros_like(value)
        else:
            out[key] = value
    return out


# ----------------------------------------------------------------------------------------------------------------------
def ensure_last_checkpoint_is_saved() -> None:
    global _PENDING
    if _PENDING is not None:
        future, finalize = _PENDING
        future.result()
        finalize()
        _PENDING = None


def _rng_state() -> dict:
    state = {"random_rng_state": random.getstate(), "np_rng_state": np.random.get_state(), "torch_rng_state": torch.get_rng_state()}
    if torch.cuda.is_available():
        state["cuda_rng_state"] = torch.cuda.get_rng_state()
    return state


def _restore_rng_state(state: dict) -> None:
    random.setstate(state["random_rng_state"])
    np.random.set_state(state["np_rng_state"])
    torch.set_rng_state(state["torch_rng_state"])
    if torch.cuda.is_available() and "cuda_rng_state" in state:
        torch.cuda.set_rng_state(state["cuda_rng_state"])


@run_rank_n
def save_args(args, save_path: str, mode: Mode | None = None) -> None:
    os.makedirs(save_path, exist_ok=True)
    with open(_training_config_path(save_path), "w") as handle:
        yaml.safe_dump(args.to_dict(), handle, indent=2, sort_keys=False)


def save_checkpoint(args, model_container, optimizer_container, lr_scheduler_container, train_dataloader,
                    experiments_tracker, iteration: int, metadata: dict | None = None) -> None:
    global _PENDING
    ensure_last_checkpoint_is_saved()
    save_path_root = args.save_args.save_path
    # everything is written into `global_step{N}.incomplete`; the directory gets its final name only when every rank
    # has written its part, so a `global_step{N}` directory that exists is always whole (a job killed mid-save
    # leaves an `.incomplete` directory that nothing reads)
    final_path = _base(save_path_root, iteration)
    save_path = final_path + ".incomplete"
    if ProcessGroupManager.get_global_rank() == 0 and os.path.isdir(save_path):
        shutil.rmtree(save_path)
    _barrier()
    os.makedirs(save_path, exist_ok=True)
    save_optimizer = args.save_args.save_optimizer and optimizer_container is not None

    if lr_scheduler_container is not None and save_optimizer:
        path = _lr_scheduler_path(save_path)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save([None if s is None else s.state_dict() for s in lr_scheduler_container], path)
    path = _rng_path(save_path)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    torch.save(_rng_state(), path)
    if train_dataloader is not None and hasattr(train_dataloader, "state_dict"):
        path = _dataloader_path(save_path)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save(train_dataloader.state_dict(), path)
    if ProcessGroupManager.get_global_rank() == 0:
        if experiments_tracker is not None:
            with open(_tracker_path(save_path), "w") as handle:
                json.dump(experiments_tracker.state_dict(), handle, indent=4)
        if metadata is not None:
            with open(_metadata_path(save_path), "w") as handle:
                json.dump(metadata, handle, indent=4)
    save_args(args, save_path)

    def finalize() -> None:
        _barrier()
        if ProcessGroupManager.get_global_rank() == 0:
            if os.path.isdir(final_path):
                shutil.rmtree(final_path)
            os.replace(save_path, final_path)
            tmp = _latest_path(save_path_root) + ".tmp"
            with open(tmp, "w") as handle:
                json.dump({"latest_checkpointed_iteration": iteration}, handle, indent=4)
            os.replace(tmp, _latest_path(save_path_root))
        if os.path.exists(os.path.join(save_path_root, _KILLSWITCH)):
            log_rank_0(logging.WARN, "KILLSWITCH found: exiting after the checkpoint")
            ProcessGroupManager.destroy_process_groups()
            sys.exit(0)

    model_state = get_model_state_dict(model_container)
    no_dist = not dist.is_initialized()
    if args.save_args.async_checkpointing:
        state = {"model": model_state}
        if save_optimizer:
            state["optimizer"] = get_optimizer_state_dict(model_container, optimizer_container)
        if no_dist:
            dcp.save({"state": state}, checkpoint_id=_model_optimizer_path(save_path), no_dist=True)
            finalize()
        else:
            future = dcp.async_save({"state": state}, checkpoint_id=_model_optimizer_path(save_path))
            _PENDING = (future, finalize)
        return
    dcp.save({"state": model_state}, checkpoint_id=_model_path(save_path), no_dist=no_dist)
    if save_optimizer:
        dcp.save({"state": get_optimizer_state_dict(model_container, optimizer_container)},
                 checkpoint_id=_optimizer_path(save_path), no_dist=no_dist)
    finalize()


def _resolve_iteration(load_path: str, iteration: int | None) -> int:
    if iteration is not None:
        return iteration
    with open(_latest_path(load_path)) as handle:
        return json.load(handle)["latest_checkpointed_iteration"]


def load_checkpoint_for_training(args, mode: Mode, model_container, optimizer_container, lr_scheduler_container,
                                 train_dataloader):
    """Returns ``(starting_iteration, metadata, experiments_tracker_state)``."""
    la = args.load_args
    if la is None or la.load_path is None:
        return 0, None, None
    iteration = _resolve_iteration(la.load_path, la.iteration)
    load_path = _base(la.load_path, iteration)
    log_rank_0(logging.INFO, f"loading checkpoint saved at {load_path}")
    no_dist = not dist.is_initialized()
    combined = os.path.isdir(_model_optimizer_path(load_path))
    load_optimizer = la.load_optimizer and optimizer_container is not None

    model_state = _placeholders(get_model_state_dict(model_container))
    if combined:
        state = {"model": model_state}
        if load_optimizer:
            _prime_optimizer_state(optimizer_container)
            state["optimizer"] = _placeholders(get_optimizer_state_dict(model_container, optimizer_container))
        dcp.load({"state": state}, checkpoint_id=_model_optimizer_path(load_path), no_dist=no_dist)
        set_model_state_dict(model_container, state["model"])
        if load_optimizer:
            set_optimizer_state_dict(model_container, optimizer_container, state["optimizer"])
    else:
        dcp.load({"state": model_state}, checkpoint_id=_model_path(load_path), no_dist=no_dist)
        set_model_state_dict(model_container, model_state)
        if load_optimizer:
            _prime_optimizer_state(optimizer_container)
            opt_state = _placeholders(get_optimizer_state_dict(model_container, optimizer_container))
            dcp.load({"state": opt_state}, checkpoint_id=_optimizer_path(load_path), no_dist=no_dist)
            set_optimizer_state_dict(model_container, optimizer_container, opt_state)
    for model in model_container:
        engine = getattr(model, "_lm_engine", None)
        if engine is not None:
            engine.refresh_parameters()

    if la.load_lr_scheduler and lr_scheduler_container is not None and os.path.exists(_lr_scheduler_path(load_path)):
        states = torch.load(_lr_scheduler_path(load_path), weights_only=False)
        for scheduler, state in zip(lr_scheduler_container, states):
            if scheduler is not None and state is not None:
                lr_lambdas = scheduler.lr_lambdas
                scheduler.load_state_dict(state)
                scheduler.lr_lambdas = lr_lambdas
    elif la.resume_learning_rate and lr_scheduler_container is not None:
        _resume_learning_rate(lr_scheduler_container, iteration)

    if la.load_rng_state and os.path.exists(_rng_path(load_path)):
        _restore_rng_state(torch.load(_rng_path(load_path), weights_only=False))
    if la.load_dataloader_state and train_dataloader is not None and os.path.exists(_dataloader_path(load_path)):
        train_dataloader.load_state_dict(torch.load(_dataloader_path(load_path), weights_only=False))

    metadata = None
    if os.path.isfile(_metadata_path(load_path)):
        with open(_metadata_path(load_path)) as handle:
            metadata = json.load(handle)
    tracker_state = None
    if la.load_experiments_tracker_state and os.path.isfile(_tracker_path(load_path)):
        with open(_tracker_path(load_path)) as handle:
            tracker_state = json.load(handle)
    starting_iteration = iteration if la.load_starting_iteration else 0
    return starting_iteration, metadata, tracker_state


def _prime_optimizer_state(optimizer_container) -> None:
    """Create the (zero) moment tensors so that a state dict with the right keys and shapes exists before loading."""
    for optimizer in optimizer_container:
        if optimizer is None:
            continue
        for group in optimizer.param_groups:
            for p in group["params"]:
                state = optimizer.state.setdefault(p, {})
                if "exp_avg" not in state:
                    state.setdefault("step", 0)
                    state["exp_avg"] = torch.zeros_like(p)
                    state["exp_avg_sq"] = torch.zeros_like(p)


def _resume_learning_rate(lr_scheduler_container, iteration: int) -> None:
    """Put freshly built schedulers at ``iteration`` (the learning rate the interrupted run would use next)."""
    for scheduler in lr_scheduler_container:
        if scheduler is None:
            continue
        scheduler.last_epoch = iteration
        for group, base_lr, fn in zip(scheduler.optimizer.param_groups, scheduler.base_lrs, scheduler.lr_lambdas):
            group["lr"] = base_lr * fn(iteration)
        scheduler._last_lr = [g["lr"] for g in scheduler.optimizer.param_groups]


def load_checkpoint_for_inference(args, mode: Mode, use_meta: bool = False):
    """Rebuild the model described by a training checkpoint on ONE process and fill it with the consolidated weights.

    Returns ``(model_wrapper, training_args, full_state_dict)``.
    """
    from ..arguments import TrainingArgs
    from ..model_wrapper import get_model_container

    la = args.load_args
    iteration = _resolve_iteration(la.load_path, la.iteration)
    load_path = _base(la.load_path, iteration)
    log_rank_0(logging.INFO, f"loading checkpoint saved at {load_path}")
    config = load_yaml(_training_config_path(load_path))
    config.pop("teacher_args", None)
    training_args = TrainingArgs(**config)
    saved_tp = training_args.distributed_args.tensor_parallel_world_size
    training_args.distributed_args.tensor_parallel_world_size = 1
    training_args.distributed_args.pipeline_parallel_world_size = 1
    training_args.distributed_args.num_pipeline_stages = 1
    if getattr(args, "mixed_precision_args", None) is not None:
        training_args.mixed_precision_args = args.mixed_precision_args

    with ProcessGroupManager.set_dummy_tensor_parallel_world_size(1), ProcessGroupManager.set_dummy_tensor_parallel_rank(0), \
            ProcessGroupManager.set_dummy_pipeline_parallel_world_size(1), ProcessGroupManager.set_dummy_pipeline_parallel_rank(0):
        container = get_model_container(training_args, Mode.inference if mode != Mode.unsharding else Mode.unsharding)
    wrapper = container[0]
    # tensors are allocated with the shapes on disk: a tensor-parallel run writes every split parameter as the
    # rank-order concatenation of its blocks (padded vocabulary, q_attn / kv_attn for multi-query attention), which
    # `fix_unsharded_state_dict` turns into the single-device layout afterwards
    combined = os.path.isdir(_model_optimizer_path(load_path))
    store = _model_optimizer_path(load_path) if combined else _model_path(load_path)
    prefix = "state.model." if combined else "state."
    saved = dcp.FileSystemReader(store).read_metadata().state_dict_metadata
    state = {k[len(prefix):]: torch.empty(tuple(v.size), dtype=torch.float32) for k, v in saved.items()
             if k.startswith(prefix) and hasattr(v, "size") and not k[len(prefix):].startswith("teacher_model.")}
    holder = {"state": {"model": state}} if combined else {"state": state}
    dcp.load(holder, checkpoint_id=store, no_dist=True)
    state = holder["state"]["model"] if combined else holder["state"]
    if saved_tp > 1:
        from ..hf_models.tp_weights import fix_unsharded_state_dict

        state = fix_unsharded_state_dict(wrapper.config, state, saved_tp, prefix="model.")
    dtype = string_to_torch_dtype(training_args.mixed_precision_args.dtype)
    state = {k: v.to(dtype) for k, v in state.items()}
    if not use_meta:
        wrapper.load_state_dict(state, strict=True)
    return wrapper, training_args, state
