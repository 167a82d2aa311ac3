"""Sharded data-parallel training engine (ZeRO 0 / 2 / 3) built for large-memory GPUs.

What the reference gets from FSDP2 ``fully_shard`` (lm_engine/distributed.py:223-308) is done here explicitly:

* Parameters of one unit (a transformer block, or everything outside the blocks) live in ONE flat buffer in the
  compute dtype; ``module.parameters()`` are views into it, so a gather fills every weight of the unit with a single
  collective and no copy-out, and kernels see plain dense tensors (no DTensor dispatch on the hot path).
* fp32 master weights, optimizer moments and (after the reduce-scatter) gradients are sharded over the ``fsdp``
  group; every rank owns one contiguous slice of each unit. Parameters of the same optimizer group are laid out
  contiguously, so a rank's slice of a group is one flat segment and the optimizer runs one fused kernel per
  segment.
* Gradients are accumulated in fp32 in a full-size buffer per unit (``param.main_grad`` views). The GEMM
  epilogues of this library add weight gradients straight into it; gradients produced by autograd are folded in
  after each micro-step. Once per optimizer step the buffer is reduce-scattered (all-reduced over the
  replication group for hybrid sharding).
* With 180 GB per GPU the gathered compute copy stays resident for the whole optimizer step (all
  gradient-accumulation micro-steps), so parameters are gathered once per step rather than twice per micro-step.
  ``resident_parameters=False`` (``distributed_args.keep_parameters_gathered: false``) instead keeps only the
  1 / N shards of every block: its parameters are all-gathered into a pooled buffer before the block's forward and
  before its backward pass and released afterwards, and its gradients are reduce-scattered right after its backward
  pass into a persistent fp32 shard, so no full-size weight copy or gradient buffer of the blocks outlives a block.

The same code runs on CPU ranks over gloo (fp32) - that is what the 2-rank loss-parity test uses.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Iterable

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops.timeline import site
from ..utils import ProcessGroupManager
from .collectives import all_gather_in_place, all_reduce_sum, reduce_scatter_in_place

_ALIGN = 128  # elements; keeps every parameter 256-byte aligned in bf16 (TMA wants 16 bytes)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class _Slot:
    name: str
    param: nn.Parameter
    shape: torch.Size
    numel: int
    offset: int
    group: str


@dataclass
class Segment:
    """This rank's slice of one optimizer group of one unit."""

    unit: "FlatUnit"
    group: str
    start: int  # offset inside the unit's local shard
    numel: int
    master: nn.Parameter = None  # fp32 view of the master shard (what the optimizer updates)
    compute: torch.Tensor | None = None  # view of the compute copy covering the same elements
    broadcast: tuple | None = None  # (address of the compute arena per rank, multicast address or 0, element offset)


class FlatUnit:
    def __init__(self, name: str, named_params: list[tuple[str, nn.Parameter]], group_of: Callable[[str, nn.Parameter], str],
                 group_order: list[str], shard_world: int, shard_rank: int, compute_dtype: torch.dtype,
                 device: torch.device, storage: Callable[[int, torch.dtype], torch.Tensor] | None = None, resident: bool = True,
                 offload: bool = False) -> None:
        self.name = name
        self.local_only = False  # True: this rank's own parameters (expert parallelism), no collective touches them
        # False: only this rank's shard of the compute copy and of the gradients is kept; the full buffers exist while
        # the unit's forward / backward pass runs (see ShardedTrainingEngine.gather_unit / release_unit)
        self.resident = resident
        # True: the fp32 master shard (and with it the optimizer's moments) and a staging copy of the gradient shard live in
        # pinned host memory; the optimizer runs on the CPU and its result is copied into the device's compute shard
        self.offload = offload
        self.module = None
        self.world = shard_world
        self.rank = shard_rank
        self.compute_dtype = compute_dtype
        self.device = device

        keyed = sorted(named_params, key=lambda kv: (group_order.index(group_of(*kv)), kv[0]))
        self.slots: list[_Slot] = []
        self.group_ranges: dict[str, tuple[int, int]] = {}
        cursor = 0
        for pname, p in keyed:
            g = group_of(pname, p)
            if g not in self.group_ranges:
                self.group_ranges[g] = (cursor, cursor)
            self.slots.append(_Slot(pname, p, p.shape, p.numel(), cursor, g))
            cursor = _round_up(cursor + p.numel(), _ALIGN)
            self.group_ranges[g] = (self.group_ranges[g][0], cursor)
        self.numel = _round_up(max(cursor, _ALIGN), _ALIGN * shard_world)
        self.shard_numel = self.numel // shard_world
        lo = self.rank * self.shard_numel
        self.shard_range = (lo, lo + self.shard_numel)

        aliased = compute_dtype == torch.float32 and not offload
        new = storage if storage is not None else (lambda n, dtype: torch.zeros(n, dtype=dtype, device=device))

        def host(n: int) -> torch.Tensor:
            t = torch.zeros(n, dtype=torch.float32)
            return t.pin_memory() if device.type == "cuda" else t

        if resident:
            self.compute = new(self.numel, compute_dtype)
            # fp32 training keeps no separate master: the shard region of the compute buffer is the master
            if offload:
                self.master = host(self.shard_numel)
            else:
                self.master = self.compute[lo : lo + self.shard_numel] if aliased else torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
            self.compute_shard = self.compute[lo : lo + self.shard_numel]
            self.grad = new(self.numel, torch.float32)
            self.grad_shard = self.grad[lo : lo + self.shard_numel]
        else:
            self.compute = None  # gathered on demand
            self.master = host(self.shard_numel) if offload else torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
            self.compute_shard = self.master if aliased else torch.zeros(self.shard_numel, dtype=compute_dtype, device=device)
            self.grad = None  # full-size only during the unit's backward pass
            self.grad_shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        self.grad_host = host(self.shard_numel) if offload else None
        self.master_is_alias = aliased

        self.segments: list[Segment] = []
        for g, (g0, g1) in self.group_ranges.items():
            s0, s1 = max(g0, lo), min(g1, lo + self.shard_numel)
            if s1 <= s0:
                continue
            seg = Segment(self, g, s0 - lo, s1 - s0)
            seg.master = nn.Parameter(self.master[seg.start : seg.start + seg.numel], requires_grad=True)
            seg.master.grad = (self.grad_host if offload else self.grad_shard)[seg.start : seg.start + seg.numel]
            seg.compute = None if aliased else self.compute_shard[s0 - lo : s1 - lo]
            seg.master._lm_engine_segment = seg
            self.segments.append(seg)

    @staticmethod
    def planned_numel(params: list[tuple[str, nn.Parameter]], shard_world: int) -> int:
        """Length of the flat buffers a unit of these parameters will have (independent of their order)."""
        cursor = 0
        for _, p in params:
            cursor = _round_up(cursor + p.numel(), _ALIGN)
        return _round_up(max(cursor, _ALIGN), _ALIGN * shard_world)

    # ------------------------------------------------------------------ parameter materialisation
    @torch.no_grad()
    def adopt(self, slot: _Slot, value_fp32: torch.Tensor) -> None:
        """Copy an initial value into the flat storage and re-point the parameter at its compute view."""
        flat = value_fp32.reshape(-1)
        slot.param._lm_engine_unit = self
        lo, hi = self.shard_range
        a, b = max(slot.offset, lo), min(slot.offset + slot.numel, hi)
        if not self.resident:
            if b > a:
                self.master[a - lo : b - lo].copy_(flat[a - slot.offset : b - slot.offset])
                if not self.master_is_alias:
                    self.compute_shard[a - lo : b - lo].copy_(flat[a - slot.offset : b - slot.offset])
            if self.compute is not None:  # adopted while gathered (checkpoint load between two passes)
                self.compute[slot.offset : slot.offset + slot.numel].copy_(flat)
            else:
                self.point_parameter_at_placeholder(slot)
            return
        self.compute[slot.offset : slot.offset + slot.numel].copy_(flat)
        if not self.master_is_alias:
            if b > a:
                self.master[a - lo : b - lo].copy_(flat[a - slot.offset : b - slot.offset])
        view = self.compute[slot.offset : slot.offset + slot.numel].view(slot.shape)
        slot.param.data = view
        slot.param.main_grad = self.grad[slot.offset : slot.offset + slot.numel].view(slot.shape)

    def point_parameter_at_placeholder(self, slot: _Slot) -> None:
        """A released parameter keeps its shape (code that only asks for sizes keeps working) but owns no memory."""
        slot.param.data = torch.empty(1, dtype=self.compute_dtype, device=self.device).expand(slot.shape)
        if hasattr(slot.param, "main_grad"):
            del slot.param.main_grad

    def full_param_fp32(self, slot: _Slot, group: dist.ProcessGroup | None) -> torch.Tensor:
        """The fp32 master value of one parameter, assembled from all shards (used for checkpoints)."""
        if self.master_is_alias and self.resident:
            return self.compute[slot.offset : slot.offset + slot.numel].view(slot.shape).float().clone()
        if self.world == 1:
            full = self.master.to(self.device)
        else:
            full = torch.empty(self.numel, dtype=torch.float32, device=self.device)
            full[self.shard_range[0] : self.shard_range[1]].copy_(self.master)
            all_gather_in_place(full, self.shard_numel, self.rank, group)
        return full[slot.offset : slot.offset + slot.numel].view(slot.shape).clone()


class ShardedTrainingEngine:
    """Owns the flat storage of a model and implements gradient reduction, clipping and parameter refresh."""

    def __init__(
        self,
        model: nn.Module,
        compute_dtype: torch.dtype = torch.float32,
        zero_stage: int = 3,
        device: torch.device | None = None,
        block_class_names: Iterable[str] | None = None,
        group_of: Callable[[str, nn.Parameter], str] | None = None,
        group_order: list[str] | None = None,
        communication_dtype: torch.dtype | None = None,
        fused_collectives: bool = True,
        frozen_prefixes: tuple[str, ...] = (),
        sequence_parallel: bool = False,
        resident_parameters: bool = True,
        cpu_offload: bool = False,
    ) -> None:
        self.model = model
        # True: fp32 master shards and optimizer state in pinned host memory, optimizer step on the CPU (what the reference
        # gets from FSDP's CPUOffloadPolicy, lm_engine/distributed.py:225 there): 12 bytes per parameter / N leave the device
        self.cpu_offload = cpu_offload
        # False: the parameters of every block exist in full only while that block runs (ZeRO-3 as the reference's
        # `reshard_after_forward`): per block an all-gather before its forward and before its backward pass and a
        # reduce-scatter of its gradients after its backward pass; between those only the 1 / N shards are held
        self.resident_parameters = resident_parameters
        self._buffer_pool: dict[tuple[int, torch.dtype], list[torch.Tensor]] = {}
        self.sequence_parallel = sequence_parallel
        self.compute_dtype = compute_dtype
        self.zero_stage = zero_stage
        self.communication_dtype = communication_dtype
        self.fused_collectives = fused_collectives
        if device is None:
            device = ProcessGroupManager.get_device() if ProcessGroupManager.is_initialized() else torch.device(
                "cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = device

        if ProcessGroupManager.is_initialized():
            self.shard_group = ProcessGroupManager.get_sharding_group()
            self.shard_world = ProcessGroupManager.get_sharding_world_size()
            self.shard_rank = ProcessGroupManager.get_sharding_rank()
            self.replica_group = ProcessGroupManager.get_replication_group()
            self.replica_world = ProcessGroupManager.get_replication_world_size()
        else:
            self.shard_group = self.replica_group = None
            self.shard_world, self.shard_rank, self.replica_world = 1, 0, 1
        self.dp_world = self.shard_world * self.replica_world
        self.tp_world = ProcessGroupManager.get_tensor_parallel_world_size() if ProcessGroupManager.is_initialized() else 1
        self.tp_group = ProcessGroupManager.get_tensor_parallel_group() if self.tp_world > 1 else None

        if group_of is None:
            from ..optimization.params_group import default_group_of

            group_of = default_group_of
        self.group_order = group_order or ["normal", "no_weight_decay", "mup"]

        block_class_names = set(block_class_names or getattr(model, "_no_split_modules", None) or ["Block"])
        self.units: list[FlatUnit] = []
        self._build_units(model, block_class_names, group_of, frozen_prefixes)
        self._grad_norm_sq = torch.zeros(1, dtype=torch.float32, device=device)
        self.clip_coef = torch.ones(1, dtype=torch.float32, device=device)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=device)
        self.micro_steps_since_reduce = 0
        # reduce-scatter of a unit as soon as its last backward of the optimizer step is done (see arm_early_reduction)
        self.early_reduction_armed = False
        self._early_reduced: set[int] = set()
        self._side_stream = None
        self._side_done = None
        for unit in self.units:
            unit.engine = self

    # ------------------------------------------------------------------ construction
    def _build_units(self, model: nn.Module, block_class_names: set[str], group_of, frozen_prefixes) -> None:
        claimed: set[int] = set()
        plan: list[tuple[str, nn.Module | None, list[tuple[str, nn.Parameter]]]] = []
        for mod_name, module in model.named_modules():
            if type(module).__name__ in block_class_names:
                params = [(f"{mod_name}.{n}", p) for n, p in module.named_parameters() if id(p) not in claimed]
                params = [(n, p) for n, p in params if p.requires_grad and not n.startswith(frozen_prefixes or ("\0",))]
                for _, p in params:
                    claimed.add(id(p))
                if params:
                    plan.append((mod_name, module, params))
        rest = [(n, p) for n, p in model.named_parameters() if id(p) not in claimed and p.requires_grad
                and not n.startswith(frozen_prefixes or ("\0",))]
        if rest:
            plan.append(("__root__", None, rest))

        # Expert-parallel parameters differ from rank to rank (every rank owns other experts) and receive the gradient
        # of all ranks' tokens through the dispatch: they get units of their own that are never reduced or gathered.
        split_plan = []
        for unit_name, module, params in plan:
            local = [(n, p) for n, p in params if getattr(p, "_expert_parallel", False)]
            shared = [(n, p) for n, p in params if not getattr(p, "_expert_parallel", False)]
            if shared:
                split_plan.append((unit_name, module, shared, False))
            if local:
                split_plan.append((unit_name + ".experts", module, local, True))

        def sharded(module, local_only) -> bool:
            return not self.resident_parameters and module is not None and not local_only and self.shard_world > 1

        if not self.resident_parameters and self.tp_world > 1:
            raise NotImplementedError("keep_parameters_gathered=False is not available together with tensor parallelism")
        storage = self._peer_storage(sum(FlatUnit.planned_numel(params, self.shard_world) for _, module, params, local in split_plan
                                         if not local and not sharded(module, local)))
        materialised: set[int] = set()
        for unit_name, module, params, local_only in split_plan:
            if local_only:
                unit = FlatUnit(unit_name, params, group_of, self.group_order, 1, 0, self.compute_dtype, self.device, None,
                                offload=self.cpu_offload)
            elif sharded(module, local_only):
                unit = FlatUnit(unit_name, params, group_of, self.group_order, self.shard_world, self.shard_rank,
                                self.compute_dtype, self.device, None, resident=False, offload=self.cpu_offload)
                unit.module = module
                self._install_gather_hooks(unit, module)
            else:
                unit = FlatUnit(unit_name, params, group_of, self.group_order, self.shard_world, self.shard_rank,
                                self.compute_dtype, self.device, storage, offload=self.cpu_offload)
            unit.local_only = local_only
            self._materialise(unit, module if id(module) not in materialised else None)
            materialised.add(id(module))
            self.units.append(unit)
            if self.peer is not None and not local_only and unit.resident and not unit.offload:
                arena = self.arenas[self.compute_dtype]
                for seg in unit.segments:
                    if seg.compute is not None:
                        # where the fused optimizer stores the updated values on every rank (element offset in the arena)
                        seg.broadcast = (arena.ptrs, arena.multicast_ptr, arena.offset_of(seg.compute) // seg.compute.element_size())
        self._materialise_buffers(model)
        sharded = [u for u in self.units if not u.resident]
        for before, after in zip(sharded[:-1], sharded[1:]):
            before.next_sharded, after.prev_sharded = after, before

    def _peer_storage(self, total_numel: int):
        """With peer-memory collectives every unit's compute and gradient buffers are slices of two symmetric arenas
        (one rendezvous each), so that kernels can address the same element on every rank. Returns the carving
        function for :class:`FlatUnit`, or ``None`` to let units allocate ordinary tensors."""
        self.peer = None
        self.arenas: dict[torch.dtype, object] = {}
        if not (self.fused_collectives and self.shard_world > 1 and self.device.type == "cuda" and self.compute_dtype != torch.float32):
            return None
        from .symmetric import get_peer_group

        self.peer = get_peer_group(self.shard_group, self.device)
        if self.peer is None:
            return None
        self.arenas = {self.compute_dtype: self.peer.alloc(total_numel, self.compute_dtype), torch.float32: self.peer.alloc(total_numel, torch.float32)}
        cursors = {dtype: 0 for dtype in self.arenas}

        def carve(numel: int, dtype: torch.dtype) -> torch.Tensor:
            start = cursors[dtype]
            cursors[dtype] = start + numel
            return self.arenas[dtype].tensor[start : start + numel]

        return carve

    @torch.no_grad()
    def _materialise(self, unit: FlatUnit, module: nn.Module | None) -> None:
        on_meta = any(s.param.is_meta for s in unit.slots)
        if on_meta:
            # Build real fp32 parameters for this unit only, initialise them, adopt them, drop the temporaries.
            owners = self._owning_modules(unit) if module is None else [module]
            for owner in owners:
                self._init_on_device(owner, unit)
        for slot in unit.slots:
            unit.adopt(slot, slot.param.data.to(device=self.device, dtype=torch.float32))

    def _owning_modules(self, unit: FlatUnit) -> list[nn.Module]:
        wanted = {id(s.param) for s in unit.slots}
        owners = []
        for module in self.model.modules():
            if any(id(p) in wanted for p in module.parameters(recurse=False)):
                owners.append(module)
        return owners

    def _init_on_device(self, owner: nn.Module, unit: FlatUnit) -> None:
        """Replace the meta parameters of ``owner`` that belong to ``unit`` by real fp32 ones and initialise them."""
        slot_of = {id(s.param): s for s in unit.slots}
        for module in owner.modules():
            direct = [(n, p) for n, p in module.named_parameters(recurse=False) if id(p) in slot_of and p.is_meta]
            if not direct:
                continue
            for n, p in direct:
                real = nn.Parameter(torch.empty(p.shape, dtype=torch.float32, device=self.device), requires_grad=p.requires_grad)
                real.__dict__.update(p.__dict__)  # optimizer-group markers travel with the parameter
                slot = slot_of.pop(id(p))
                self._replace_parameter(p, real)
                slot.param = real
                slot_of[id(real)] = slot
            if hasattr(module, "reset_parameters"):
                module.reset_parameters()
            else:
                raise RuntimeError(f"{type(module).__name__} has parameters on the meta device but no reset_parameters()")

    def _replace_parameter(self, old: nn.Parameter, new: nn.Parameter) -> None:
        for module in self.model.modules():
            for name, p in list(module._parameters.items()):
                if p is old:
                    module._parameters[name] = new

    @torch.no_grad()
    def _materialise_buffers(self, model: nn.Module) -> None:
        for module in model.modules():
            buffers = list(module.named_buffers(recurse=False))
            if not buffers:
                continue
            if any(b.is_meta for _, b in buffers):
                if hasattr(module, "reset_parameters") and not any(True for _ in module.parameters(recurse=False)):
                    module.reset_parameters()
                    for name, b in list(module.named_buffers(recurse=False)):
                        module._buffers[name] = b.to(self.device)
                else:
                    raise RuntimeError(f"cannot materialise buffers of {type(module).__name__}")
            else:
                for name, b in buffers:
                    module._buffers[name] = b.to(self.device)

    # ------------------------------------------------------------------ parameters that exist in full only while used
    def _take_buffer(self, numel: int, dtype: torch.dtype, stream=None) -> torch.Tensor:
        """A pooled buffer; the stream that is going to use it first waits for the buffer's last user."""
        free = self._buffer_pool.setdefault((numel, dtype), [])
        if not free:
            return torch.empty(numel, dtype=dtype, device=self.device)
        buf, last_use = free.pop()
        if last_use is not None:
            (stream if stream is not None else torch.cuda.current_stream()).wait_event(last_use)
        return buf

    def _give_buffer(self, buf: torch.Tensor) -> None:
        last_use = None
        if self.device.type == "cuda":
            last_use = torch.cuda.Event()
            last_use.record()  # on the current stream: whoever used the buffer last
        self._buffer_pool.setdefault((buf.numel(), buf.dtype), []).append((buf, last_use))

    def _collective_stream(self):
        """Side stream of the sharded-parameter mode: gathers of the next block and reductions of the previous one run
        here, under the compute of the current block (CUDA only; CPU ranks run everything in order)."""
        if self.device.type != "cuda":
            return None
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device, priority=-1)
        return self._side_stream

    @torch.no_grad()
    def start_gather(self, unit: "FlatUnit | None") -> None:
        """Begin the all-gather of a sharded unit on the side stream (no-op on CPU, for resident or already gathered
        units). ``gather_unit`` picks the result up."""
        side = self._collective_stream()
        if unit is None or side is None or unit.resident or unit.compute is not None or getattr(unit, "pending_gather", None) is not None:
            return
        buf = self._take_buffer(unit.numel, self.compute_dtype, stream=side)
        now = torch.cuda.Event()
        now.record()  # the shard was last written by the optimizer on the compute stream
        side.wait_event(now)
        with torch.cuda.stream(side):
            lo, hi = unit.shard_range
            buf[lo:hi].copy_(unit.compute_shard)
            all_gather_in_place(buf, unit.shard_numel, unit.rank, self.shard_group)
            done = torch.cuda.Event()
            done.record()
        unit.pending_gather = (buf, done)

    @torch.no_grad()
    def gather_unit(self, unit: FlatUnit, for_backward: bool = False) -> None:
        """Make the full parameters of a sharded unit available (all-gather of the ranks' shards into a pooled
        buffer, possibly started earlier on the side stream); for a backward pass also a zeroed full-size fp32 gradient
        buffer behind ``param.main_grad``."""
        if unit.resident:
            return
        if unit.compute is None:
            pending = getattr(unit, "pending_gather", None)
            if pending is not None:
                buf, done = pending
                torch.cuda.current_stream().wait_event(done)
                unit.pending_gather = None
            else:
                buf = self._take_buffer(unit.numel, self.compute_dtype)
                lo, hi = unit.shard_range
                buf[lo:hi].copy_(unit.compute_shard)
                all_gather_in_place(buf, unit.shard_numel, unit.rank, self.shard_group)
            unit.compute = buf
            for slot in unit.slots:
                slot.param.data = buf[slot.offset : slot.offset + slot.numel].view(slot.shape)
        if for_backward and unit.grad is None:
            unit.grad = self._take_buffer(unit.numel, torch.float32).zero_()
            for slot in unit.slots:
                slot.param.main_grad = unit.grad[slot.offset : slot.offset + slot.numel].view(slot.shape)

    @torch.no_grad()
    def release_unit(self, unit: FlatUnit) -> None:
        """Give the full buffers back. Gradients of the pass that just ended are summed over the ranks first and this
        rank's slice is added to its persistent gradient shard (on the side stream where there is one, so that the
        reduction runs under the backward pass of the next block)."""
        if unit.resident:
            return
        if unit.grad is not None:
            for slot in unit.slots:  # gradients that autograd left in .grad join the buffer before it is reduced
                g = slot.param.grad
                if g is not None:
                    slot.param.main_grad.add_(g.to(torch.float32))
                    slot.param.grad = None
            side = self._collective_stream()
            if side is None:
                reduced = reduce_scatter_in_place(unit.grad, unit.shard_numel, unit.rank, self.shard_group, False)
                unit.grad_shard.add_(reduced)
                self._give_buffer(unit.grad)
            else:
                ready = torch.cuda.Event()
                ready.record()  # every gradient of the unit is in the buffer (and older clears of the shard are done)
                side.wait_event(ready)
                with torch.cuda.stream(side):
                    reduced = reduce_scatter_in_place(unit.grad, unit.shard_numel, unit.rank, self.shard_group, False)
                    unit.grad_shard.add_(reduced)
                    self._give_buffer(unit.grad)
                    self._side_done = torch.cuda.Event()
                    self._side_done.record()
            unit.grad = None
            for slot in unit.slots:
                if hasattr(slot.param, "main_grad"):
                    del slot.param.main_grad
        if unit.compute is not None:
            self._give_buffer(unit.compute)
            unit.compute = None
        for slot in unit.slots:
            unit.point_parameter_at_placeholder(slot)

    def _install_gather_hooks(self, unit: FlatUnit, module: nn.Module) -> None:
        unit.in_backward = False

        def before_forward(mod, args):
            self.gather_unit(unit)
            self.start_gather(getattr(unit, "next_sharded", None))  # the next block's weights arrive under this block's compute

        def after_forward(mod, args, output):
            if unit.in_backward:  # a forward pass re-run inside the backward pass (activation checkpointing) keeps them
                return
            if torch.is_grad_enabled() and getattr(unit, "next_sharded", None) is None:
                return  # the last block is the first one the backward pass needs: keep it
            self.release_unit(unit)

        def before_backward(mod, grad_output):
            unit.in_backward = True
            self.gather_unit(unit, for_backward=True)
            self.start_gather(getattr(unit, "prev_sharded", None))

        def after_backward(mod, grad_input, grad_output):
            unit.in_backward = False
            self.release_unit(unit)

        module.register_forward_pre_hook(before_forward)
        module.register_forward_hook(after_forward)
        module.register_full_backward_pre_hook(before_backward)
        module.register_full_backward_hook(after_backward)

    # ------------------------------------------------------------------ views for the optimizer
    def segments(self) -> list[Segment]:
        return [seg for unit in self.units for seg in unit.segments]

    def segments_by_group(self) -> dict[str, list[Segment]]:
        out: dict[str, list[Segment]] = {}
        for seg in self.segments():
            out.setdefault(seg.group, []).append(seg)
        return out

    def named_slots(self):
        for unit in self.units:
            for slot in unit.slots:
                yield unit, slot

    def num_parameters(self) -> int:
        return sum(slot.numel for _, slot in self.named_slots())

    # ------------------------------------------------------------------ gradient path
    @torch.no_grad()
    def fold_autograd_grads(self) -> None:
        """Add gradients that autograd left in ``param.grad`` into the fp32 accumulation buffers."""
        for unit, slot in self.named_slots():
            g = slot.param.grad
            if g is None:
                continue
            if not unit.resident and not hasattr(slot.param, "main_grad"):
                raise RuntimeError(f"{slot.name}: a gradient arrived after the unit's gradients were reduced and released")
            if g.is_cuda and g.dtype == torch.bfloat16 and ops.native_available() and g.is_contiguous():
                ops.native().cast_bf16_to_f32(g.view(-1), slot.param.main_grad.view(-1), True, 1.0)
            else:
                slot.param.main_grad.add_(g.to(torch.float32))
            slot.param.grad = None
        self.micro_steps_since_reduce += 1

    @torch.no_grad()
    def zero_grad(self) -> None:
        for unit in self.units:
            (unit.grad if unit.resident else unit.grad_shard).zero_()

    # ------------------------------------------------------------------ reduction under the last backward pass
    def arm_early_reduction(self) -> bool:
        """Call before the LAST micro-step of an optimizer step. From then on a unit whose backward pass reports itself
        finished (``unit_backward_done``) is reduce-scattered at once on a side stream, under the backward pass of the
        units below it, so that only the units that finish last (the first block, the embeddings) are reduced in the
        open after the backward pass. Needs the peer-memory collectives; returns whether it is active."""
        import os

        self.early_reduction_armed = (self.peer is not None and self.tp_world == 1 and self.replica_world == 1
                                      and os.environ.get("LM_ENGINE_OVERLAP_REDUCE", "1") != "0")
        return self.early_reduction_armed

    @torch.no_grad()
    def unit_backward_done(self, unit: "FlatUnit") -> None:
        """Every gradient of ``unit`` for this optimizer step is in its fp32 buffer (called by the backward pass of the
        unit's last micro-step, on the compute stream)."""
        if not self.early_reduction_armed or unit.local_only or not unit.resident or id(unit) in self._early_reduced:
            return
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device, priority=-1)
        ready = torch.cuda.Event()
        ready.record()
        self._side_stream.wait_event(ready)
        with torch.cuda.stream(self._side_stream):
            # all ranks have this unit's gradients complete; then each sums its slice of all copies
            self.peer.side_barrier()
            self.peer.reduce_scatter_f32(self.arenas[torch.float32], unit.grad_shard, unit.grad_shard)
        self._early_reduced.add(id(unit))

    @torch.no_grad()
    def reduce_gradients(self) -> None:
        """Sum gradients over the data parallel ranks; afterwards ``unit.grad_shard`` holds this rank's slice. Under
        tensor parallelism the partial gradients of replicated parameters are first summed over that group."""
        if self.tp_world > 1:
            from ..hf_models.models.tensor_parallel import reduce_tensor_parallel_grads

            reduce_tensor_parallel_grads(self.model, self.sequence_parallel)
        if self.peer is not None:
            # every rank has finished its backward pass; then each sums its own slice of all copies; then nobody
            # clears or refills its copy before the others have read it
            arena = self.arenas[torch.float32]
            if self._early_reduced:
                with site("step.wait_for_early_reduce_scatter"):
                    done = torch.cuda.Event()
                    done.record(self._side_stream)
                    torch.cuda.current_stream().wait_event(done)
            with site("step.barrier_before_reduce_scatter"):
                self.peer.barrier()
            with site("step.reduce_scatter"):
                for unit in self.units:
                    if not unit.local_only and unit.resident and id(unit) not in self._early_reduced:
                        self.peer.reduce_scatter_f32(arena, unit.grad_shard, unit.grad_shard)
            with site("step.barrier_after_reduce_scatter"):
                self.peer.barrier()
            self._early_reduced.clear()
            self.early_reduction_armed = False
        for unit in self.units:
            if unit.local_only:
                continue
            if not unit.resident:
                self.release_unit(unit)  # normally done by the backward hook already
                if self._side_done is not None:
                    torch.cuda.current_stream().wait_event(self._side_done)  # the unit's reduction on the side stream
            elif self.shard_world > 1 and self.peer is None:
                reduce_scatter_in_place(unit.grad, unit.shard_numel, unit.rank, self.shard_group, False)
            if self.replica_world > 1:
                all_reduce_sum(unit.grad_shard, self.replica_group)
        self.micro_steps_since_reduce = 0

    @torch.no_grad()
    def grad_norm_sq(self) -> torch.Tensor:
        """Squared norm of the summed gradient held by this engine's ranks (all data- and tensor-parallel ranks of
        one pipeline stage), after :meth:`reduce_gradients`. Every parameter counts once."""
        native = ops.native_available() and self.device.type == "cuda"
        total = self._grad_norm_sq
        if native:
            C = ops.native()
            first = True
            for unit in self.units:
                C.sumsq(unit.grad_shard, total, not first)
                first = False
        else:
            total.zero_()
            for unit in self.units:
                total.add_(unit.grad_shard.double().pow(2).sum().float())
        replicated = None
        if self.tp_world > 1:
            # parameters replicated over the tensor-parallel group count once, the sharded ones once per rank
            replicated = self._replicated_grad_norm_sq()
            total.sub_(replicated)
            if self.shard_world > 1:
                all_reduce_sum(replicated, self.shard_group)
        if self.shard_world > 1:
            all_reduce_sum(total, self.shard_group)
        if self.tp_world > 1:
            all_reduce_sum(total, self.tp_group)
            total.add_(replicated)
        return total

    @torch.no_grad()
    def clip_grad_norm(self, max_norm: float | None, extra_norm_groups: list | None = None,
                       precomputed_norm_sq: torch.Tensor | None = None) -> torch.Tensor:
        """Global gradient norm of the averaged gradient; sets ``self.clip_coef`` (device scalar) for the optimizer.

        Gradients in the buffers are SUMS over data parallel ranks; the averaging factor ``1 / dp_world`` is applied
        here and inside the optimizer, never by rewriting the buffers. ``precomputed_norm_sq`` carries a squared norm
        that already covers more than this engine (all pipeline stages).
        """
        if precomputed_norm_sq is None:
            total = self.grad_norm_sq()
            for group in extra_norm_groups or []:
                all_reduce_sum(total, group)
        else:
            total = precomputed_norm_sq
        norm = total.sqrt() * (1.0 / self.dp_world)
        self.grad_norm.copy_(norm)
        if max_norm is not None and max_norm > 0:
            self.clip_coef.copy_((max_norm / (norm + 1e-6)).clamp(max=1.0))
        else:
            self.clip_coef.fill_(1.0)
        return self.grad_norm

    def _replicated_grad_norm_sq(self) -> torch.Tensor:
        """Squared gradient norm of this rank's shard elements that belong to parameters without a tensor-parallel
        split (identical on every rank of that group after :meth:`reduce_gradients`)."""
        out = torch.zeros(1, dtype=torch.float32, device=self.device)
        for unit in self.units:
            lo, hi = unit.shard_range
            for slot in unit.slots:
                if getattr(slot.param, "_tp_shard_dim", None) is not None:
                    continue
                a, b = max(slot.offset, lo), min(slot.offset + slot.numel, hi)
                if b > a:
                    out += unit.grad_shard[a - lo : b - lo].double().pow(2).sum().float()
        return out

    @property
    def grad_mul(self) -> float:
        return 1.0 / self.dp_world

    # ------------------------------------------------------------------ parameter refresh
    @torch.no_grad()
    def refresh_parameters(self, masters_already_cast: bool = False, broadcast_done: bool = False) -> None:
        """After the optimizer step: cast updated masters into the compute copy and gather the other shards."""
        broadcast_by_optimizer = masters_already_cast and broadcast_done and self.peer is not None
        for unit in self.units:
            if not unit.master_is_alias and not masters_already_cast:
                dst = unit.compute_shard
                if dst.is_cuda and unit.master.is_cuda and ops.native_available() and dst.dtype == torch.bfloat16:
                    ops.native().cast_f32_to_bf16(unit.master, dst)
                else:
                    dst.copy_(unit.master)
        if self.shard_world > 1 and not broadcast_by_optimizer:
            if self.peer is not None:
                arena = self.arenas[self.compute_dtype]
                self.peer.barrier()
                for unit in self.units:
                    if not unit.local_only and unit.resident:
                        self.peer.all_gather(arena, unit.compute, unit.shard_numel)
            else:
                for unit in self.units:
                    if not unit.local_only and unit.resident:
                        all_gather_in_place(unit.compute, unit.shard_numel, unit.rank, self.shard_group, False)
        if self.peer is not None:
            self.peer.barrier()  # every rank's stores into this rank's copy have landed before the next forward pass

    # ------------------------------------------------------------------ one optimizer step
    @torch.no_grad()
    def optimizer_step(self, optimizer, lr_scheduler=None, max_norm: float | None = None,
                       extra_norm_groups: list | None = None, precomputed_norm_sq: torch.Tensor | None = None) -> torch.Tensor:
        """Reduce gradients, clip, update the fp32 shards, refresh the compute copy. Returns the gradient norm
        (a device scalar; nothing here synchronises with the host)."""
        if precomputed_norm_sq is None:
            self.reduce_gradients()
        with site("step.grad_norm"):
            grad_norm = self.clip_grad_norm(max_norm, extra_norm_groups, precomputed_norm_sq)
        fused = getattr(optimizer, "writes_compute_copy", False)
        if fused:
            optimizer.grad_scale = self.clip_coef
            optimizer.grad_mul = self.grad_mul
        else:
            factor = self.clip_coef * self.grad_mul
            for unit in self.units:
                unit.grad_shard.mul_(factor.to(unit.grad_shard.device))
        with site("step.adamw(+broadcast)"):
            if self.cpu_offload:
                # reduced, unscaled gradient shards to pinned host memory; the optimizer (clip coefficient and 1 / dp
                # applied there) then runs on the CPU and copies its result into the device's compute shard
                for unit in self.units:
                    unit.grad_host.copy_(unit.grad_shard, non_blocking=True)
                if self.device.type == "cuda":
                    torch.cuda.current_stream(self.device).synchronize()
            optimizer.step()
        if lr_scheduler is not None:
            lr_scheduler.step()
        with site("step.refresh_parameters"):
            self.refresh_parameters(masters_already_cast=fused, broadcast_done=fused and getattr(optimizer, "last_step_broadcast", False))
        if fused and not self.cpu_offload and (self.shard_world == 1 or all(not u.resident or u.local_only for u in self.units)):
            pass  # the fused kernel cleared every gradient element it consumed
        else:
            with site("step.zero_grad"):
                self.zero_grad()
        return grad_norm

    # ------------------------------------------------------------------ state dicts (full, fp32, by parameter name)
    @torch.no_grad()
    def full_state_dict(self, prefix: str = "") -> dict[str, torch.Tensor]:
        out = {}
        for unit, slot in self.named_slots():
            out[prefix + slot.name] = unit.full_param_fp32(slot, self.shard_group)
        return out

    @torch.no_grad()
    def load_full_state_dict(self, state: dict[str, torch.Tensor], prefix: str = "", strict: bool = True) -> None:
        for unit, slot in self.named_slots():
            key = prefix + slot.name
            if key not in state:
                if strict:
                    raise KeyError(f"missing parameter {key}")
                continue
            unit.adopt(slot, state[key].to(device=self.device, dtype=torch.float32))

    def memory_summary(self) -> dict[str, float]:
        gib = 1 / 2**30
        width = torch.empty((), dtype=self.compute_dtype).element_size()
        compute = sum((u.numel if u.resident else u.shard_numel) * width for u in self.units)
        grads = sum((u.numel if u.resident else u.shard_numel) * 4 for u in self.units)
        master = sum(0 if u.master_is_alias else u.master.numel() * 4 for u in self.units)
        return {"compute_GiB": compute * gib, "grad_GiB": grads * gib, "master_GiB": master * gib}
