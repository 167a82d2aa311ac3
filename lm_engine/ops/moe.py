"""Mixture-of-experts expert computation on grouped rows (the role ScatterMoE plays for the reference, see
lm_engine/hf_models/modeling_utils/mlp_blocks/moe.py:262-291 there).

Token copies are laid out grouped by expert; every expert's range starts at a multiple of 128 rows and is zero-padded
to the next multiple, so each 128-row GEMM tile belongs to one expert and nothing about the launch depends on the
routing outcome (no host synchronisation). One layer is

    gather rows -> grouped GEMM (c_fc) -> SwiGLU -> grouped GEMM (c_proj) -> weighted combine per token

with an explicit backward that recomputes the activation from the saved c_fc output instead of saving it. Under
expert parallelism the same kernels read token rows / expert outputs directly from the peers' buffers (see
:mod:`lm_engine.parallel.expert_parallel`).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .timeline import site

from . import _weight_grad_target, native, native_available, status_word

TILE = 128


@dataclass
class GroupedLayout:
    """Placement of ``entries`` (token, slot) pairs into expert-grouped, tile-padded rows."""

    dest_row: torch.Tensor  # int32 [entries]: row of each entry (-1: not placed here)
    src_entry: torch.Tensor  # int32 [rows]: entry held by each row (-1: padding)
    tile_expert: torch.Tensor  # int32 [rows / 128]: expert of each tile (>= num_experts: unused tile)
    padded_offsets: torch.Tensor  # int32 [num_experts + 1]
    rows: int  # static upper bound, multiple of 128
    dropped: torch.Tensor | None = None  # int32 [1]: entries that did not fit under a capacity bound (device counter)


def worst_case_rows(entries: int, num_local_experts: int) -> int:
    return ((entries + num_local_experts * (TILE - 1)) + TILE - 1) // TILE * TILE


def build_grouped_layout(expert_of_entry: torch.Tensor, num_experts: int, first_expert: int = 0,
                         num_local_experts: int | None = None, capacity_rows: int | None = None) -> GroupedLayout:
    """Stable counting sort of entries by expert with tile-aligned expert ranges, on the device (no host sync).

    ``expert_of_entry``: int [entries]. Entries whose expert is outside ``[first_expert, first_expert + local)`` are not
    placed (their ``dest_row`` is -1), which is how one rank of an expert parallel group selects its share.
    ``capacity_rows`` bounds the row buffer below the worst case (all entries on this rank); entries that do not fit are
    dropped and counted in ``dropped``. On a GPU the layout comes from three small kernels (``csrc/ops/moe_layout.cu``);
    the torch formulation below is the reference and the CPU path, and gives the same result element for element.
    """
    local = num_experts if num_local_experts is None else num_local_experts
    entries = expert_of_entry.numel()
    device = expert_of_entry.device
    rows = worst_case_rows(entries, local)
    if capacity_rows is not None:
        rows = min(rows, max(TILE, (capacity_rows + TILE - 1) // TILE * TILE))
    if expert_of_entry.is_cuda and local <= 256 and native_available() and hasattr(native(), "moe_layout"):
        flat = expert_of_entry.reshape(-1).to(torch.int32).contiguous()
        dest_row, src_entry, tile_expert, padded_offsets, dropped = native().moe_layout(flat, first_expert, local, rows)
        return GroupedLayout(dest_row, src_entry, tile_expert, padded_offsets, rows, dropped)
    e = expert_of_entry.reshape(-1).to(torch.int64) - first_expert
    mine = (e >= 0) & (e < local)
    key = torch.where(mine, e, torch.full_like(e, local))  # foreign entries sort last
    order = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=local + 1)[:local]
    padded = (counts + TILE - 1) // TILE * TILE
    padded_end = torch.cumsum(padded, 0)
    padded_start = padded_end - padded
    start = torch.cumsum(counts, 0) - counts

    sorted_key = key[order]
    placed = sorted_key < local
    safe_key = sorted_key.clamp(max=local - 1)
    position = torch.arange(entries, device=device) - start[safe_key]
    row_sorted = torch.where(placed, padded_start[safe_key] + position, torch.full_like(position, -1))
    fits = row_sorted < rows
    dropped = (placed & ~fits).sum().to(torch.int32).reshape(1)
    placed = placed & fits
    row_sorted = torch.where(placed, row_sorted, torch.full_like(row_sorted, -1))
    padded_start = padded_start.clamp(max=rows)
    padded_end = padded_end.clamp(max=rows)

    dest_row = torch.empty(entries, dtype=torch.int32, device=device)
    dest_row[order] = row_sorted.to(torch.int32)
    src_entry = torch.full((rows + 1,), -1, dtype=torch.int32, device=device)
    src_entry[torch.where(placed, row_sorted, torch.full_like(row_sorted, rows))] = order.to(torch.int32)
    src_entry = src_entry[:rows].contiguous()

    tile_start = torch.arange(rows // TILE, device=device) * TILE
    tile_expert = torch.searchsorted(padded_end, tile_start, right=True).to(torch.int32)  # == local for unused tiles
    padded_offsets = torch.cat([padded_start.new_zeros(1), padded_end]).to(torch.int32)
    return GroupedLayout(dest_row, src_entry, tile_expert, padded_offsets, rows, dropped)


def build_group_layout(expert_of_entry: torch.Tensor, num_experts: int, experts_per_owner: int, owner: int,
                       capacity_rows: int | None = None) -> tuple[GroupedLayout, torch.Tensor | None]:
    """`build_grouped_layout` for rank ``owner`` of an expert-parallel group whose ranks each own ``experts_per_owner``
    consecutive experts, plus, for EVERY entry of the routing table, the row it gets on its own owner as
    ``owner * rows + row`` (-1 if dropped there). Every rank holds the same table and the same ``rows``, so every rank
    arrives at the same numbers and nothing has to be exchanged. Without the kernel the second value is ``None``."""
    entries = expert_of_entry.numel()
    rows = worst_case_rows(entries, experts_per_owner)
    if capacity_rows is not None:
        rows = min(rows, max(TILE, (capacity_rows + TILE - 1) // TILE * TILE))
    if expert_of_entry.is_cuda and num_experts <= 256 and native_available() and hasattr(native(), "moe_layout_group"):
        flat = expert_of_entry.reshape(-1).to(torch.int32).contiguous()
        dest_row, src_entry, tile_expert, padded_offsets, dropped, global_row = native().moe_layout_group(
            flat, num_experts, experts_per_owner, owner, rows)
        return GroupedLayout(dest_row, src_entry, tile_expert, padded_offsets, rows, dropped), global_row
    layout = build_grouped_layout(expert_of_entry, num_experts, first_expert=owner * experts_per_owner,
                                  num_local_experts=experts_per_owner, capacity_rows=capacity_rows)
    return layout, None


def native_moe_ok(x: torch.Tensor, activation_function: str) -> bool:
    return (native_available() and x.is_cuda and x.dtype == torch.bfloat16 and activation_function == "swiglu"
            and x.shape[-1] % 8 == 0 and hasattr(native(), "grouped_rows"))


def fused_dispatch_enabled(C) -> bool:
    """Gather inside the grouped GEMM kernel (on unless ``LM_ENGINE_MOE_FUSED_DISPATCH=0``)."""
    import os

    return hasattr(C, "grouped_rows_dispatch") and os.environ.get("LM_ENGINE_MOE_FUSED_DISPATCH", "1") != "0"


def gather_then_grouped_rows(C, src_ptrs, src_entry, hidden, entries_per_rank, top_k, like, tile_expert, owners, weight, w_mn, st,
                             copy_ctas: int = 32, out=None):
    """``rows = gather(src)[src_entry]; out = rows @ op(weight[expert of the tile])`` -> ``(rows, out)``. One kernel when
    the fused dispatch is available (gather CTAs feed the GEMM CTAs tile by tile), otherwise the gather kernel followed by
    the grouped GEMM."""
    if fused_dispatch_enabled(C) and hidden * 2 <= 16384:
        return C.grouped_rows_dispatch(src_ptrs, src_entry, entries_per_rank, top_k, weight, tile_expert, w_mn, st, copy_ctas, out)
    rows = C.moe_gather(src_ptrs, [], src_entry, hidden, entries_per_rank, top_k, like, tile_expert, owners)
    return rows, C.grouped_rows(rows, weight, tile_expert, w_mn, st, out)


def _wgrad(C, dy, x, weight, padded_offsets, st):
    target = _weight_grad_target(weight)
    if target is not None:
        C.grouped_wgrad(dy, x, target.view(weight.shape), padded_offsets, True, st)
        return None
    dw = torch.zeros(weight.shape, device=weight.device, dtype=torch.float32)
    C.grouped_wgrad(dy, x, dw, padded_offsets, False, st)
    return dw.to(weight.dtype)


def weighted_swiglu_backward(C, fc, dact, dest_row, entry_weights, rows: int, tile_expert, owners: int):
    """One pass over the expert rows: the routing-weighted activation ``w * swiglu(fc)`` (operand of the second
    weight gradient), ``dfc`` (gradient of the first GEMM's output, routing weight folded in) and, per routed entry,
    ``<dact_row, swiglu(fc)_row>`` = the gradient of its routing weight (0 for entries without a row here)."""
    served = dest_row >= 0
    safe = torch.where(served, dest_row, torch.full_like(dest_row, rows)).long()
    row_weight = torch.zeros(rows + 1, dtype=torch.float32, device=fc.device)
    row_weight[safe] = entry_weights
    act_w, dfc, dot = C.moe_swiglu_bwd(fc, dact, row_weight[:rows], tile_expert, owners)
    per_entry = torch.cat([dot, dot.new_zeros(1)])[safe]
    return act_w, dfc, per_entry


class _ScatteredExpertsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_fc, w_proj, router_weights, selected_experts, num_experts, top_k):
        C = native()
        st = status_word(x.device)
        T, H = x.shape
        with site("moe.fwd.layout"):
            layout = build_grouped_layout(selected_experts.reshape(-1), num_experts)
        te = layout.tile_expert  # tiles past the used rows carry num_experts and are skipped by every kernel below
        with site("moe.fwd.gather+c_fc"):
            xg, fc = gather_then_grouped_rows(C, [x.data_ptr()], layout.src_entry, H, T * top_k, top_k, x, te, num_experts, w_fc, False, st)
        with site("moe.fwd.swiglu"):
            act = C.swiglu_fwd(fc, te, num_experts)
        with site("moe.fwd.c_proj"):
            y = C.grouped_rows(act, w_proj, layout.tile_expert, False, st)
        del act
        weights32 = router_weights.reshape(-1).float().contiguous()
        with site("moe.fwd.combine"):
            out = C.moe_combine([y.data_ptr()], layout.dest_row, weights32, T, H, top_k, layout.rows, x)
        # the gathered rows are kept for the weight gradient of c_fc (one [rows, H] buffer per layer instead of a second gather)
        ctx.save_for_backward(x, w_fc, w_proj, weights32, fc, layout.dest_row, layout.src_entry, layout.tile_expert, layout.padded_offsets, xg)
        ctx.meta = (num_experts, top_k, layout.rows, router_weights.dtype, router_weights.shape)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w_fc, w_proj, weights32, fc, dest_row, src_entry, tile_expert, padded_offsets, xg = ctx.saved_tensors
        num_experts, top_k, rows, w_dtype, w_shape = ctx.meta
        C = native()
        st = status_word(x.device)
        T, H = x.shape
        dout = dout.contiguous()
        entries = T * top_k

        # dY of the second GEMM without the routing weight, and the activation recomputed from the saved c_fc output
        with site("moe.bwd.gather+c_proj.dgrad"):
            dyg, dact = gather_then_grouped_rows(C, [dout.data_ptr()], src_entry, H, entries, top_k, x, tile_expert, num_experts, w_proj, True, st)  # [rows, I] = dyg @ w_proj[e]
        with site("moe.bwd.swiglu"):
            act, dfc, per_entry = weighted_swiglu_backward(C, fc, dact, dest_row, weights32, rows, tile_expert, num_experts)
        del dact
        d_weights = per_entry.view(w_shape).to(w_dtype)
        with site("moe.bwd.c_proj.wgrad"):
            g_proj = _wgrad(C, dyg, act, w_proj, padded_offsets, st)  # dW2[e] = dyg^T (w * act)
        del dyg, act
        with site("moe.bwd.c_fc.wgrad"):
            g_fc = _wgrad(C, dfc, xg, w_fc, padded_offsets, st)
        with site("moe.bwd.c_fc.dgrad"):
            dxg = C.grouped_rows(dfc, w_fc, tile_expert, True, st)  # [rows, H] = dfc @ w_fc[e]
        with site("moe.bwd.combine"):
            dx = C.moe_combine([dxg.data_ptr()], dest_row, None, T, H, top_k, rows, x)
        return dx, g_fc, g_proj, d_weights, None, None, None


def scattered_experts_mlp(x: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor, router_weights: torch.Tensor,
                          selected_experts: torch.Tensor, num_experts: int, top_k: int, activation_function: str) -> torch.Tensor:
    """``sum_s router_weights[t, s] * c_proj[e](swiglu(c_fc[e](x[t])))`` with ``e = selected_experts[t, s]``."""
    assert activation_function == "swiglu"
    return _ScatteredExpertsFn.apply(x.contiguous(), w_fc, w_proj, router_weights, selected_experts, num_experts, top_k)
