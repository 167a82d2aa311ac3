"""Expert parallelism: every rank of the group owns ``num_experts / ep`` experts and serves the tokens of all ranks.

The reference has no expert parallelism (its MoE is sharded by FSDP or sliced by tensor parallelism); this is the
engine's own design for NVLink domains. Dispatch and combine are not all-to-all collectives: token rows stay where they
were produced, in symmetric memory, and the kernels that feed and drain the grouped GEMMs read them from there.

forward, on every rank (T local tokens, k experts per token, E_local local experts):
  1. all-gather of the routing decisions (``[ep, T, k]`` expert ids and weights: a few hundred KB, NCCL)
  2. layout of the (token, slot) entries of ALL ranks that picked a local expert: expert-grouped rows, every expert
     padded to a multiple of 128 rows (device ops only, static upper bound on the row count)
  3. ``moe_gather`` pulls those token rows from the owners' activations through peer pointers (dispatch)
  4. grouped tcgen05 GEMM (c_fc) -> SwiGLU -> grouped GEMM (c_proj), output rows in symmetric memory
  5. all-to-all of the row numbers (int32) so that every token owner knows where its k results are
  6. ``moe_combine`` sums the k rows of each local token straight from the owners' output buffers, weighted (combine)
backward mirrors it: the output gradient is pulled like the tokens, the input gradient combined like the outputs, and
the gradient of the routing weights travels back with one small all-to-all. Bounded peer barriers order the phases.

On CPU (and for tensors the kernels do not take) ``expert_parallel_mlp`` falls back to a differentiable gather ->
local experts -> reduce-scatter over the group with the same results, which is what the gloo tests run.
"""

from __future__ import annotations

import os

import torch

from ..ops.timeline import site
import torch.distributed as dist

from .. import ops
from ..ops.moe import TILE, _wgrad, build_group_layout, build_grouped_layout, gather_then_grouped_rows, weighted_swiglu_backward, worst_case_rows
from ..utils import ProcessGroupManager
from .symmetric import PeerBuffer, PeerGroup, get_peer_group

_WORKSPACES: dict[int, "_Workspace"] = {}

# Sizing of the per-rank row buffers (expert inputs, projections, outputs):
#   None (default)  exact and dropless: every rank derives, from the routing table it already holds for the whole group,
#                   the tile-padded row count of the fullest rank and reads it back (one small device-to-host read per
#                   MoE layer and forward pass); buffers then hold what the busiest rank needs, nothing is ever dropped.
#                   The size actually used is the largest need seen so far in the run (all layers share it) plus one
#                   eighth of headroom when it grows, rounded up to `_ROW_QUANTUM`: a buffer size that changed with every batch and layer kept the caching allocator
#                   mapping new memory in the middle of the run (stalls of about a second at 4 GPUs), a size that only
#                   ever grows settles after a few steps
#   a factor >= 1   static bound without a host read: ``factor x (a rank's balanced share of the routed entries)`` rows
#                   (plus tile padding); entries beyond it are dropped (they contribute nothing to their token) and
#                   counted on the device in ``_DROPPED``
_CAPACITY_FACTOR: float | None = None
# CTAs of the fused dispatch + GEMM kernel that pull rows from the peers (each keeps about 190 KB in flight)
_GATHER_CTAS = int(os.environ.get("LM_ENGINE_MOE_GATHER_CTAS", "32"))
_DROPPED: dict[torch.device, torch.Tensor] = {}
_ROW_QUANTUM = 2048
_ROW_HIGH_WATER: dict[tuple, int] = {}  # (device, routed entries of the group, local experts) -> rows


def set_expert_capacity_factor(factor: float | None) -> None:
    global _CAPACITY_FACTOR
    assert factor is None or factor >= 1.0, "expert_capacity_factor must be at least 1"
    _CAPACITY_FACTOR = factor


def dropped_entries(device: torch.device) -> int:
    """Entries dropped on this rank since the start of the run (synchronises with the device)."""
    counter = _DROPPED.get(device)
    return 0 if counter is None else int(counter.item())


def _capacity_rows(entries_per_rank: int, local_experts: int) -> int | None:
    if _CAPACITY_FACTOR is None:
        return None
    return int(_CAPACITY_FACTOR * entries_per_rank + 0.5) + local_experts * (TILE - 1)


class _RowCount:
    """Exact sizing: the tile-padded row count of the fullest rank, computed on the device from the routing table that
    every rank holds for the whole group (so all ranks get the same number) and copied to pinned host memory without
    blocking. ``value()`` waits for that copy only: whatever was queued behind it keeps the GPU busy meanwhile."""

    def __init__(self, selected_all: torch.Tensor, num_experts: int, local_experts: int) -> None:
        counts = torch.zeros(num_experts, dtype=torch.int32, device=selected_all.device)
        counts.index_add_(0, selected_all, torch.ones_like(selected_all))
        padded = (counts + (TILE - 1)) // TILE * TILE
        fullest = padded.view(-1, local_experts).sum(dim=1).max().to(torch.int32).reshape(1)
        self.host = torch.empty(1, dtype=torch.int32, pin_memory=True)
        self.host.copy_(fullest, non_blocking=True)
        self.ready = torch.cuda.Event()
        self.ready.record()

    def value(self) -> int:
        self.ready.synchronize()
        return max(TILE, int(self.host[0]))


def _count_dropped(layout) -> None:
    if _CAPACITY_FACTOR is None or layout.dropped is None:
        return
    device = layout.dropped.device
    if device not in _DROPPED:
        _DROPPED[device] = torch.zeros(1, dtype=torch.int64, device=device)
    _DROPPED[device] += layout.dropped


def ep_world() -> int:
    return ProcessGroupManager.get_expert_parallel_world_size() if ProcessGroupManager.is_initialized() else 1


def ep_rank() -> int:
    return ProcessGroupManager.get_expert_parallel_rank() if ProcessGroupManager.is_initialized() else 0


def ep_group():
    return ProcessGroupManager.get_expert_parallel_group()


# ----------------------------------------------------------------------------------------------------------------------
# reference path: plain collectives, any device
class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        pieces = [torch.empty_like(x) for _ in range(ep_world())]
        dist.all_gather(pieces, x.contiguous(), group=ep_group())
        return torch.cat(pieces, dim=0)

    @staticmethod
    def backward(ctx, g):
        total = g.contiguous().clone()
        dist.all_reduce(total, group=ep_group())
        return total.chunk(ep_world(), dim=0)[ep_rank()].contiguous()


class _ScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        total = x.contiguous().clone()
        dist.all_reduce(total, group=ep_group())
        return total.chunk(ep_world(), dim=0)[ep_rank()].contiguous()

    @staticmethod
    def backward(ctx, g):
        pieces = [torch.empty_like(g) for _ in range(ep_world())]
        dist.all_gather(pieces, g.contiguous(), group=ep_group())
        return torch.cat(pieces, dim=0)


def _reference(x, w_fc, w_proj, b_fc, b_proj, weights, selected, num_experts, activation):
    local = w_fc.shape[0]
    first = ep_rank() * local
    x_all = _GatherRows.apply(x)
    weights_all = _GatherRows.apply(weights)
    selected_all = torch.cat(_all_gather_plain(selected), dim=0)
    out = torch.zeros_like(x_all)
    for e in range(local):
        token, slot = torch.where(selected_all == first + e)
        if token.numel() == 0:
            continue
        h = torch.nn.functional.linear(x_all[token], w_fc[e], None if b_fc is None else b_fc[e])
        h = torch.nn.functional.linear(activation(h), w_proj[e], None if b_proj is None else b_proj[e])
        out = out.index_add(0, token, h * weights_all[token, slot].unsqueeze(-1))
    return _ScatterRows.apply(out)


def _all_gather_plain(t: torch.Tensor) -> list[torch.Tensor]:
    pieces = [torch.empty_like(t) for _ in range(ep_world())]
    dist.all_gather(pieces, t.contiguous(), group=ep_group())
    return pieces


# ----------------------------------------------------------------------------------------------------------------------
# peer-memory path
class _Workspace:
    """Symmetric buffers of one expert-parallel group, shared by all layers (they run one after the other)."""

    def __init__(self, peer: PeerGroup) -> None:
        self.peer = peer
        self.tokens: PeerBuffer | None = None  # [T, H] rows this rank owns (activations, or their gradients)
        self.rows: PeerBuffer | None = None  # [rows, H] rows this rank computed (expert outputs, or input gradients)

    def buffer(self, attr: str, numel: int) -> PeerBuffer:
        buf = getattr(self, attr)
        if buf is None or buf.tensor.numel() < numel:
            buf = self.peer.alloc(numel, torch.bfloat16, zero=False)
            setattr(self, attr, buf)
        return buf


def workspace(device: torch.device) -> _Workspace | None:
    key = id(ep_group())
    if key not in _WORKSPACES:
        peer = get_peer_group(ep_group(), device)
        _WORKSPACES[key] = None if peer is None else _Workspace(peer)
    return _WORKSPACES[key]


def _exchange_rows(dest_row: torch.Tensor, entries: int, rows: int) -> torch.Tensor:
    """``dest_row``: for all ``ep * entries`` global entries, the row on THIS rank (-1 if another rank's expert).
    Returns for this rank's ``entries`` the global row ``owner * rows + row`` on the owner."""
    world = ep_world()
    received = torch.empty_like(dest_row)
    dist.all_to_all_single(received, dest_row.contiguous(), group=ep_group())
    received = received.view(world, entries)
    owner = received.argmax(dim=0)  # exactly one owner reports a row >= 0
    local = received.max(dim=0).values
    # an entry that its owner had to drop (capacity bound) has no row anywhere: -1, which the combine kernel skips
    return torch.where(local >= 0, owner.to(torch.int32) * rows + local, torch.full_like(local, -1)).to(torch.int32).contiguous()


def _exchange_values(per_entry: torch.Tensor, entries: int) -> torch.Tensor:
    """Sum over owners of a per-entry fp32 value computed for all global entries (zero where not owned)."""
    received = torch.empty_like(per_entry)
    dist.all_to_all_single(received, per_entry.contiguous(), group=ep_group())
    return received.view(ep_world(), entries).sum(dim=0)


class _ExpertParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_fc, w_proj, router_weights, selected_experts, num_experts, top_k):
        C = ops.native()
        st = ops.status_word(x.device)
        ws = workspace(x.device)
        peer = ws.peer
        world, rank = peer.world, peer.rank
        T, H = x.shape
        local = w_fc.shape[0]
        entries = T * top_k

        with site("ep.fwd.routing_all_gather"):
            # one collective for the routing table of the whole group: expert ids and the bit patterns of the fp32 weights
            mine = torch.cat([selected_experts.reshape(-1).to(torch.int32), router_weights.reshape(-1).float().view(torch.int32)])
            table = torch.empty(world, 2 * entries, dtype=torch.int32, device=x.device)
            dist.all_gather_into_tensor(table, mine, group=ep_group())
            selected_all = table[:, :entries].reshape(-1)
            weights_all = table[:, entries:].reshape(-1).view(torch.float32)
            exact = _RowCount(selected_all, num_experts, local) if _CAPACITY_FACTOR is None else None
        tokens = ws.buffer("tokens", T * H)
        with site("ep.fwd.token_copy+barriers"):
            peer.barrier()  # the previous users of the buffers are done everywhere
            tokens.tensor[: T * H].view(T, H).copy_(x)
            peer.barrier()  # every rank's tokens are readable
        with site("ep.fwd.row_count_wait+layout"):
            if exact is not None:
                need = (exact.value() + _ROW_QUANTUM - 1) // _ROW_QUANTUM * _ROW_QUANTUM
                key = (x.device, world * entries, local)  # the same on every rank, like the count itself
                capacity_rows = _ROW_HIGH_WATER.get(key, 0)
                if need > capacity_rows:
                    # one eighth of headroom, so that the next slightly larger batch does not grow the buffers again
                    capacity_rows = (need + need // 8 + _ROW_QUANTUM - 1) // _ROW_QUANTUM * _ROW_QUANTUM
                    _ROW_HIGH_WATER[key] = capacity_rows
            else:
                capacity_rows = _capacity_rows(entries, local)
            layout, global_rows = build_group_layout(selected_all, num_experts, local, rank, capacity_rows)
        _count_dropped(layout)
        rows = layout.rows
        # the shared row buffer is sized for the worst case once: with exact sizing `rows` changes with every batch, and
        # growing a symmetric allocation in the middle of a run is a rendezvous of the whole group
        out_rows = ws.buffer("rows", worst_case_rows(world * entries, local) * H)
        te = layout.tile_expert  # tiles past the used rows carry `local` and are skipped by every kernel below
        # dispatch: rows are pulled from their owners by gather CTAs inside the c_fc GEMM kernel
        with site("ep.fwd.dispatch+c_fc"):
            xg, fc = gather_then_grouped_rows(C, tokens.ptrs, layout.src_entry, H, entries, top_k, x, te, local, w_fc, False, st, copy_ctas=_GATHER_CTAS)
        with site("ep.fwd.swiglu"):
            act = C.swiglu_fwd(fc, te, local)
        with site("ep.fwd.c_proj"):
            C.grouped_rows(act, w_proj, layout.tile_expert, False, st, out_rows.tensor[: rows * H].view(rows, H))  # straight into symmetric memory
        del act
        with site("ep.fwd.row_exchange+barrier"):
            if global_rows is not None:  # worked out locally from the routing table of the whole group
                global_row = global_rows[rank * entries : (rank + 1) * entries].contiguous()
            else:
                global_row = _exchange_rows(layout.dest_row, entries, rows)
            peer.barrier()  # every rank's expert outputs are readable
        weights32 = router_weights.reshape(-1).float().contiguous()
        with site("ep.fwd.combine"):
            out = C.moe_combine(out_rows.ptrs, global_row, weights32, T, H, top_k, rows, x)  # combine: pull the k results per token

        # the gathered rows are kept for the weight gradient: pulling them from the peers a second time costs more than the memory
        ctx.save_for_backward(x, w_fc, w_proj, weights_all, fc, layout.dest_row, layout.src_entry, layout.tile_expert,
                              layout.padded_offsets, global_row, xg)
        ctx.meta = (num_experts, top_k, rows, router_weights.dtype, router_weights.shape)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w_fc, w_proj, weights_all, fc, dest_row, src_entry, tile_expert, padded_offsets, global_row, xg = ctx.saved_tensors
        num_experts, top_k, rows, w_dtype, w_shape = ctx.meta
        C = ops.native()
        st = ops.status_word(x.device)
        ws = workspace(x.device)
        peer = ws.peer
        T, H = x.shape
        entries = T * top_k
        tokens = ws.buffer("tokens", T * H)
        out_rows = ws.buffer("rows", rows * H)  # the forward pass made it large enough for any batch

        with site("ep.bwd.token_copy+barriers"):
            peer.barrier()
            tokens.tensor[: T * H].view(T, H).copy_(dout)
            peer.barrier()
        local = w_fc.shape[0]
        # output gradients of the rows computed here, pulled inside the GEMM kernel as in the forward pass
        with site("ep.bwd.dispatch+c_proj.dgrad"):
            dyg, dact = gather_then_grouped_rows(C, tokens.ptrs, src_entry, H, entries, top_k, x, tile_expert, local, w_proj, True, st, copy_ctas=_GATHER_CTAS)
        # gradient of the routing weight of every entry served here (0 elsewhere), sent back to the token owners
        with site("ep.bwd.swiglu"):
            act, dfc, per_entry = weighted_swiglu_backward(C, fc, dact, dest_row, weights_all, rows, tile_expert, local)
        del dact
        with site("ep.bwd.routing_gradient_exchange"):
            d_weights = _exchange_values(per_entry, entries).view(w_shape).to(w_dtype)
        with site("ep.bwd.c_proj.wgrad"):
            g_proj = _wgrad(C, dyg, act, w_proj, padded_offsets, st)
        del dyg, act

        with site("ep.bwd.c_fc.wgrad"):
            g_fc = _wgrad(C, dfc, xg, w_fc, padded_offsets, st)
        with site("ep.bwd.c_fc.dgrad"):
            C.grouped_rows(dfc, w_fc, tile_expert, True, st, out_rows.tensor[: rows * H].view(rows, H))
        with site("ep.bwd.barrier+combine"):
            peer.barrier()
            dx = C.moe_combine(out_rows.ptrs, global_row, None, T, H, top_k, rows, x)
        return dx, g_fc, g_proj, d_weights, None, None, None


def native_ok(x: torch.Tensor, w_fc: torch.Tensor, activation_function: str, has_bias: bool) -> bool:
    from ..ops.moe import native_moe_ok

    return (not has_bias and native_moe_ok(x, activation_function) and w_fc.dtype == torch.bfloat16 and x.dim() == 2
            and hasattr(ops.native(), "peer_barrier") and workspace(x.device) is not None)


def expert_parallel_mlp(x: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor, b_fc, b_proj, router_weights: torch.Tensor,
                        selected_experts: torch.Tensor, num_experts: int, top_k: int, activation_function: str, activation) -> torch.Tensor:
    """``sum_s router_weights[t, s] * expert[selected[t, s]](x[t])`` where the experts live on the ranks of the
    expert-parallel group (``w_fc`` / ``w_proj`` hold this rank's ``num_experts / ep``)."""
    if native_ok(x, w_fc, activation_function, b_fc is not None):
        return _ExpertParallelFn.apply(x.contiguous(), w_fc, w_proj, router_weights, selected_experts, num_experts, top_k)
    return _reference(x, w_fc, w_proj, b_fc, b_proj, router_weights, selected_experts, num_experts, activation)
