"""The kernels behind the multi-GPU collectives, exercised on ONE GPU.

Every one of them addresses the other ranks through a table of device pointers, so ``world`` buffers of this GPU can
stand in for the ranks' buffers (plain loads and stores, no multicast address). Each emulated rank's kernel is launched
on its own, one after the other: none of these kernels waits for another launch (the cross-rank barrier kernel, which
does, is not part of this file). Results are compared with plain PyTorch fp32 arithmetic over the same buffers.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from lm_engine.ops.build import load_extension

    return load_extension()


def _status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_reduce_scatter_sums_every_ranks_copy(C, world):
    torch.manual_seed(0)
    n = 1 << 16  # shard elements
    copies = [torch.randn(n * world, device="cuda") for _ in range(world)]
    expected = torch.stack(copies).sum(0)
    ptrs = [c.data_ptr() for c in copies]
    for rank in range(world):
        out = torch.empty(n, device="cuda")
        C.peer_reduce_scatter_f32(ptrs, 0, out, rank * n, 0.5)
        torch.testing.assert_close(out, 0.5 * expected[rank * n : (rank + 1) * n], atol=1e-5, rtol=1e-5)
    # in place into the rank's own region, the way the training engine uses it
    snapshot = [c.clone() for c in copies]
    for rank in range(world):
        C.peer_reduce_scatter_f32(ptrs, 0, copies[rank][rank * n : (rank + 1) * n], rank * n, 1.0)
    for rank in range(world):
        torch.testing.assert_close(copies[rank][rank * n : (rank + 1) * n], expected[rank * n : (rank + 1) * n], atol=1e-5, rtol=1e-5)
        other = (rank + 1) % world
        assert torch.equal(copies[rank][other * n : (other + 1) * n], snapshot[rank][other * n : (other + 1) * n])


@pytest.mark.parametrize("world", [2, 8])
def test_all_gather_pulls_the_other_shards(C, world):
    torch.manual_seed(1)
    n = 1 << 15
    shards = [torch.randn(n, device="cuda").bfloat16() for _ in range(world)]
    copies = [torch.zeros(n * world, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    for rank in range(world):
        copies[rank][rank * n : (rank + 1) * n].copy_(shards[rank])
    ptrs = [c.data_ptr() for c in copies]
    for rank in range(world):
        C.peer_all_gather(ptrs, rank, n * 2, copies[rank])
    for rank in range(world):
        assert torch.equal(copies[rank], torch.cat(shards))


@pytest.mark.parametrize("world", [2, 4])
def test_adamw_with_broadcast_matches_the_local_update(C, world):
    torch.manual_seed(2)
    n = 1 << 14
    targets = [torch.zeros(n * world, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    ptrs = [t.data_ptr() for t in targets]
    scale = torch.full((1,), 0.5, device="cuda")
    expected = []
    for rank in range(world):
        p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        m, v = torch.rand(n, device="cuda") * 0.1, torch.rand(n, device="cuda") * 0.1
        p2, g2, m2, v2 = p.clone(), g.clone(), m.clone(), v.clone()
        local = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        C.adamw_step(p2, m2, v2, g2, local, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, scale, 0.25, True)
        C.adamw_step_bcast(p, m, v, g, ptrs, 0, rank * n, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, scale, 0.25, True)
        assert torch.equal(p, p2) and torch.equal(m, m2) and torch.equal(v, v2) and float(g.abs().max()) == 0.0
        expected.append(local)
    for rank in range(world):
        assert torch.equal(targets[rank], torch.cat(expected))


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("w_mn", [False, True])
def test_all_gather_fused_into_the_gemm(C, world, w_mn):
    torch.manual_seed(3)
    rows, K, N = 256, 512, 384
    total = rows * world
    parts = [torch.randn(rows, K, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * K**-0.5
    w_in = w.t().contiguous() if w_mn else w
    ref = torch.cat(parts).float() @ w.float().t()
    ptrs = [p.data_ptr() for p in parts]
    for rank in range(world):
        staging = torch.zeros(total, K, device="cuda", dtype=torch.bfloat16)
        staging[rank * rows : (rank + 1) * rows].copy_(parts[rank])
        ready = torch.zeros(total // 128, dtype=torch.int32, device="cuda")
        out = torch.empty(total, N, device="cuda", dtype=torch.bfloat16)
        st = _status()
        C.ag_gemm(ptrs, staging, ready, 1, w_in, out, w_mn, rank, 4, st)
        torch.cuda.synchronize()
        assert st.item() == 0
        assert torch.equal(staging, torch.cat(parts))  # the gathered rows are kept for the weight gradient
        assert _rel_err(out, ref) < 6e-3


@pytest.mark.parametrize("world", [2, 4])
def test_reduce_scatter_fused_into_the_gemm(C, world):
    torch.manual_seed(4)
    M, K, N = 512, 256, 384
    rows = M // world
    xs = [torch.randn(M, K, device="cuda", dtype=torch.bfloat16) for _ in range(world)]  # every rank's partial-sum operand
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * K**-0.5 for _ in range(world)]
    slots = [torch.zeros(world, rows, N, device="cuda", dtype=torch.bfloat16) for _ in range(world)]  # slots[r][source]
    ptrs = [s.data_ptr() for s in slots]
    for rank in range(world):
        st = _status()
        C.gemm_rs(xs[rank], ws[rank], ptrs, False, rank, st)
        torch.cuda.synchronize()
        assert st.item() == 0
    full = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    for rank in range(world):
        summed = C.sum_slots(slots[rank], world)
        assert _rel_err(summed, full[rank * rows : (rank + 1) * rows]) < 8e-3


@pytest.mark.parametrize("world", [2, 4])
def test_expert_combine_pulls_rows_through_the_pointer_table(C, world):
    torch.manual_seed(5)
    T, H, k, rows_per_rank = 300, 256, 4, 512
    outputs = [torch.randn(rows_per_rank, H, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    global_row = torch.randint(0, world * rows_per_rank, (T * k,), device="cuda", dtype=torch.int32)
    weights = torch.rand(T * k, device="cuda")
    everything = torch.cat(outputs).float()
    picked = everything[global_row.long()].view(T, k, H)
    like = outputs[0]
    out = C.moe_combine([o.data_ptr() for o in outputs], global_row, weights, T, H, k, rows_per_rank, like)
    assert _rel_err(out, (picked * weights.view(T, k, 1)).sum(1)) < 5e-3
    out = C.moe_combine([o.data_ptr() for o in outputs], global_row, None, T, H, k, rows_per_rank, like)
    assert _rel_err(out, picked.sum(1)) < 5e-3
