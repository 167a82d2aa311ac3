"""Fused all-gather+GEMM and GEMM+reduce-scatter against NCCL + fp32 matmul, on every visible GPU (torchrun, one rank
per GPU, world = tensor-parallel size). Also prints event timings of the fused kernels and of the unfused pair
(NCCL collective + this engine's GEMM). Prints ``FUSED_TP_OK`` on rank 0."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from lm_engine import ops
from lm_engine.parallel import fused_tp
from lm_engine.parallel import tensor_parallel as tp
from lm_engine.utils import init_distributed


def reference_gather_linear(x_local, w):
    x = tp._all_gather(x_local, 0).float()
    return x @ w.float().t()


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end) / iters], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def main():
    world = int(os.environ["WORLD_SIZE"])
    os.environ["LM_ENGINE_FUSED_TP"] = "1"
    init_distributed(tensor_parallel_world_size=world)
    rank = dist.get_rank()
    device = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(11 + rank)
    C = ops.native()
    st = ops.status_word(device)

    for rows, k, n in ((256, 512, 768), (1024, 4096, 3072), (512, 1536, 520)):
        x_local = (torch.randn(rows, k, device=device) * 0.5).bfloat16().requires_grad_(True)
        torch.manual_seed(5)  # the weight slice differs per rank in a real model; any values do here
        w = (torch.randn(n, k, device=device) * 0.05).bfloat16().requires_grad_(True)
        assert fused_tp.fused_ok(x_local, w, rows * world)
        y = fused_tp.ag_linear(x_local, w)
        ref = reference_gather_linear(x_local.detach(), w.detach())
        torch.testing.assert_close(y.float(), ref, atol=0.06, rtol=0.02)
        dy = (torch.randn(rows * world, n, device=device) * 0.1).bfloat16()
        y.backward(dy)
        # dx_local = reduce_scatter(dy @ w); dw = dy^T @ gather(x)
        full_dx = dy.float() @ w.detach().float()
        dist.all_reduce(full_dx)
        torch.testing.assert_close(x_local.grad.float(), full_dx[rank * rows : (rank + 1) * rows], atol=0.08, rtol=0.03)
        ref_dw = dy.float().t() @ tp._all_gather(x_local.detach(), 0).float()
        torch.testing.assert_close(w.grad.float(), ref_dw, atol=0.5, rtol=0.03)

        # row-parallel: x [T, k_local] @ w[n, k_local]^T summed over ranks, this rank keeps its rows
        x2 = (torch.randn(rows * world, k, device=device) * 0.5).bfloat16().requires_grad_(True)
        w2 = (torch.randn(n, k, device=device) * 0.05).bfloat16().requires_grad_(True)
        y2 = fused_tp.linear_rs(x2, w2)
        full = x2.detach().float() @ w2.detach().float().t()
        dist.all_reduce(full)
        torch.testing.assert_close(y2.float(), full[rank * rows : (rank + 1) * rows], atol=0.12, rtol=0.03)
        dy2 = (torch.randn(rows, n, device=device) * 0.1).bfloat16()
        y2.backward(dy2)
        dy2_full = tp._all_gather(dy2, 0).float()
        torch.testing.assert_close(x2.grad.float(), dy2_full @ w2.detach().float(), atol=0.06, rtol=0.03)
        torch.testing.assert_close(w2.grad.float(), dy2_full.t() @ x2.detach().float(), atol=0.5, rtol=0.03)
        ops.check_status()
        if rank == 0:
            print(f"numerics ok rows/rank={rows} k={k} n={n}", flush=True)

    # timings at a training-like shape: 8192 tokens in total, hidden 4096
    total, hidden = 8192, 4096
    rows = total // world
    ws = fused_tp.workspace()
    for name, n, k in (("c_attn", 6144 // world, hidden), ("c_fc", 28672 // world, hidden)):
        x_local = torch.randn(rows, k, device=device).bfloat16()
        w = torch.randn(n, k, device=device).bfloat16()
        out = torch.empty(total, n, device=device, dtype=torch.bfloat16)
        gathered = torch.empty(total, k, device=device, dtype=torch.bfloat16)

        def unfused():
            dist.all_gather_into_tensor(gathered, x_local)
            C.gemm(gathered, w, out, False, False, False, 1.0, st, 0, 0)

        def gemm_only():
            C.gemm(gathered, w, out, False, False, False, 1.0, st, 0, 0)

        t_fused, t_unfused, t_gemm = timed(lambda: ws.gather_gemm(x_local, w, False)), timed(unfused), timed(gemm_only)
        if rank == 0:
            print(f"ag_gemm {name}: fused {t_fused:.3f} ms | nccl all-gather + gemm {t_unfused:.3f} ms | gemm alone {t_gemm:.3f} ms", flush=True)
    for name, n, k in (("attn c_proj", hidden, hidden // world), ("mlp c_proj", hidden, 14336 // world)):
        x = torch.randn(total, k, device=device).bfloat16()
        w = torch.randn(n, k, device=device).bfloat16()
        partial = torch.empty(total, n, device=device, dtype=torch.bfloat16)
        scattered = torch.empty(rows, n, device=device, dtype=torch.bfloat16)

        def unfused():
            C.gemm(x, w, partial, False, False, False, 1.0, st, 0, 0)
            dist.reduce_scatter_tensor(scattered, partial)

        def gemm_only():
            C.gemm(x, w, partial, False, False, False, 1.0, st, 0, 0)

        t_fused, t_unfused, t_gemm = timed(lambda: ws.gemm_scatter(x, w, False)), timed(unfused), timed(gemm_only)
        if rank == 0:
            print(f"gemm_rs {name}: fused {t_fused:.3f} ms | gemm + nccl reduce-scatter {t_unfused:.3f} ms | gemm alone {t_gemm:.3f} ms", flush=True)
    ws.peer.check()
    ops.check_status()
    dist.barrier()
    if rank == 0:
        print("FUSED_TP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
