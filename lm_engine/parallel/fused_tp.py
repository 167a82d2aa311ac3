"""Sequence-parallel linears whose collective runs inside the GEMM kernel (``csrc/comm/tp_gemm.cu``).

``ag_linear``    ``y[T, N] = gather(x_local)[T, K] @ w^T``: gather CTAs pull the other ranks' rows over NVLink into a
                 local staging buffer while the tensor-core CTAs already work on this rank's rows.
``linear_rs``    ``y_local[T / tp, N] = reduce_scatter(x[T, K] @ w^T)``: the epilogue stores bf16 fragments into the
                 owner rank's slot for this source rank; each rank then sums its slots in fp32.

Both are differentiable; each backward is the other kernel on the transposed weight plus a weight-gradient GEMM that
accumulates into ``weight.main_grad`` when the training engine provides it. This is the role async tensor parallelism
plays in the reference (symmetric-memory micro-pipelining chosen by Inductor, lm_engine/hf_models/modeling_utils_TP/
linear.py:48-49, 104-105, 167-168 there), written as two kernels.

Buffers live in one workspace per tensor-parallel group and grow on demand; every call is bracketed by the bounded peer
barrier (inputs visible before the kernel, buffers reusable after it).
"""

from __future__ import annotations

import torch

from .. import ops
from . import tensor_parallel as tp
from .symmetric import PeerBuffer, PeerGroup, get_peer_group

ROW_BLOCK = 128
_WORKSPACES: dict[int, "_Workspace"] = {}


class _Workspace:
    def __init__(self, peer: PeerGroup) -> None:
        self.peer = peer
        self.x_sym: PeerBuffer | None = None  # this rank's rows, readable by the others (bf16)
        self.out_sym: PeerBuffer | None = None  # reduce-scatter target: one bf16 slot per source rank
        self.staging: torch.Tensor | None = None  # gathered rows (bf16)
        self.ready = torch.zeros(1 << 16, dtype=torch.int32, device=peer.device)
        self.epoch = 0
        self.copy_ctas = 16

    def _grow(self, attr: str, numel: int, dtype: torch.dtype) -> PeerBuffer:
        buf = getattr(self, attr)
        if buf is None or buf.tensor.numel() < numel:
            # symmetric allocation is collective; all ranks see the same sizes, so they grow together
            buf = self.peer.alloc(numel, dtype, zero=False)
            setattr(self, attr, buf)
        return buf

    def gather_gemm(self, x_local: torch.Tensor, w: torch.Tensor, w_mn: bool) -> tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(y, gathered x)``; the gathered rows stay valid until the next call."""
        peer, world, rank = self.peer, self.peer.world, self.peer.rank
        rows, k = x_local.shape
        total = rows * world
        n = w.shape[1] if w_mn else w.shape[0]
        x_sym = self._grow("x_sym", rows * k, torch.bfloat16)
        if self.staging is None or self.staging.numel() < total * k:
            self.staging = torch.empty(total * k, dtype=torch.bfloat16, device=x_local.device)
        staging = self.staging[: total * k].view(total, k)
        peer.barrier()  # nobody still reads the previous contents of x_sym
        x_sym.tensor[: rows * k].view(rows, k).copy_(x_local)
        staging[rank * rows : (rank + 1) * rows].copy_(x_local)
        peer.barrier()  # every rank's rows are in place
        self.epoch += 1
        y = torch.empty(total, n, dtype=torch.bfloat16, device=x_local.device)
        ops.native().ag_gemm(x_sym.ptrs, staging, self.ready, self.epoch, w, y, w_mn, rank, self.copy_ctas, ops.status_word(x_local.device))
        return y, staging

    def gemm_scatter(self, x: torch.Tensor, w: torch.Tensor, w_mn: bool) -> torch.Tensor:
        peer, world, rank = self.peer, self.peer.world, self.peer.rank
        total, _ = x.shape
        rows = total // world
        n = w.shape[1] if w_mn else w.shape[0]
        out_sym = self._grow("out_sym", world * rows * n, torch.bfloat16)
        peer.barrier()  # every rank has summed its slots of the previous call
        ops.native().gemm_rs(x, w, out_sym.ptrs, w_mn, rank, ops.status_word(x.device))
        peer.barrier()  # every rank's partial results have landed in this rank's slots
        return ops.native().sum_slots(out_sym.tensor[: world * rows * n].view(world, rows, n), world)


def workspace() -> _Workspace | None:
    group = tp.tp_group()
    key = id(group)
    if key not in _WORKSPACES:
        device = torch.device("cuda", torch.cuda.current_device())
        peer = get_peer_group(group, device)
        _WORKSPACES[key] = None if peer is None else _Workspace(peer)
    return _WORKSPACES[key]


def fused_ok(x: torch.Tensor, weight: torch.Tensor, rows_total: int) -> bool:
    """Asynchronous tensor parallelism switched on, bf16 CUDA matrices, whole 128-row blocks per rank, dimensions the
    kernels accept, peer memory available."""
    from ..utils import ProcessGroupManager

    world = tp.tp_world()
    if not ProcessGroupManager.is_async_tensor_parallel_enabled():
        return False
    if world == 1 or not ops.native_available() or not x.is_cuda or x.dim() != 2:
        return False
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or rows_total % (ROW_BLOCK * world) != 0:
        return False
    if x.shape[1] % 8 or weight.shape[0] % 8 or weight.shape[1] % 8 or not hasattr(ops.native(), "ag_gemm"):
        return False
    return workspace() is not None


def _wgrad(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor):
    """``dW[N, K] = dy[T, N]^T @ x[T, K]`` accumulated into ``weight.main_grad`` when present (returns None then)."""
    C = ops.native()
    st = ops.status_word(dy.device)
    target = getattr(weight, "main_grad", None)
    if target is not None:
        C.gemm(dy, x, target, True, True, True, 1.0, st, 0, 0)
        return None
    dw = torch.empty(weight.shape, dtype=torch.float32, device=dy.device)
    C.gemm(dy, x, dw, True, True, False, 1.0, st, 0, 0)
    return dw.to(weight.dtype)


class _GatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight):
        y, _ = workspace().gather_gemm(x_local.contiguous(), weight, False)
        ctx.save_for_backward(x_local, weight)
        return y

    @staticmethod
    def backward(ctx, dy):
        x_local, weight = ctx.saved_tensors
        ws = workspace()
        dy = dy.contiguous()
        dx_local = ws.gemm_scatter(dy, weight, True)  # (dy @ W)[rows of this rank], summed over ranks
        # the weight gradient needs the gathered input again; only the local rows were kept for the backward pass
        gathered = tp._all_gather(x_local.contiguous(), 0)
        dw = _wgrad(dy, gathered, weight)
        return dx_local, dw


class _LinearScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return workspace().gemm_scatter(x.contiguous(), weight, False)

    @staticmethod
    def backward(ctx, dy_local):
        x, weight = ctx.saved_tensors
        dx, dy_full = workspace().gather_gemm(dy_local.contiguous(), weight, True)  # gather(dy) @ W
        dw = _wgrad(dy_full, x.contiguous(), weight)
        return dx, dw


def ag_linear(x_local: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    y = _GatherLinear.apply(x_local, weight)
    return y if bias is None else y + bias


def linear_rs(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return _LinearScatter.apply(x, weight)
