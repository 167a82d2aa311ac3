"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op."""

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


def _worst_row_err(a, b):
    """Largest relative error of any single row (a whole-tensor norm can hide one bad row among thousands)."""
    a, b = a.float().reshape(-1, a.shape[-1]), b.float().reshape(-1, b.shape[-1])
    return ((a - b).norm(dim=-1) / (b.norm(dim=-1) + 1e-3 * b.norm() / b.shape[0] ** 0.5 + 1e-12)).max().item()


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (200, 264, 136), (1000, 72, 328), (520, 1032, 2048)])
def test_gemm_layouts(C, a_mn, b_mn, shape, variant):
    M, N, K = shape
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    st = _status()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm(a_in, b_in, out, a_mn, b_mn, False, 1.0, st, 0, variant)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert _rel_err(out, ref) < 6e-3
    out32 = torch.empty(M, N, device="cuda", dtype=torch.float32)
    C.gemm(a_in, b_in, out32, a_mn, b_mn, False, 0.5, st, 0, variant)
    assert _rel_err(out32, 0.5 * ref) < 1e-5
    base = torch.randn(M, N, device="cuda", dtype=torch.float32)
    acc = base.clone()
    C.gemm(a_in, b_in, acc, a_mn, b_mn, True, 1.0, st, 0, variant)
    assert _rel_err(acc, base + ref) < 1e-5
    assert st.item() == 0


@pytest.mark.parametrize("variant", [1, 2])
def test_gemm_persistent_many_tiles(C, variant):
    torch.manual_seed(1)
    M, N, K = 4096, 4096, 1024
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    st = _status()
    C.gemm(a, b, out, False, False, False, 1.0, st, 0, variant)
    ref = (a.float() @ b.float().t())
    assert st.item() == 0
    assert _rel_err(out, ref) < 6e-3
    out2 = torch.empty_like(out)
    C.gemm(a, b, out2, False, False, False, 1.0, st, 0, variant)
    assert torch.equal(out, out2)  # run-to-run determinism


def test_gemm_strided_views(C):
    torch.manual_seed(2)
    big = torch.randn(300, 1024, device="cuda", dtype=torch.bfloat16)
    a = big[:, 256:768]  # row stride 1024, 512 wide
    w = torch.randn(384, 512, device="cuda", dtype=torch.bfloat16)
    outbuf = torch.zeros(300, 1024, device="cuda", dtype=torch.bfloat16)
    out = outbuf[:, 128:512]
    st = _status()
    C.gemm(a, w, out, False, False, False, 1.0, st, 0)
    assert st.item() == 0
    assert _rel_err(out, a.float() @ w.float().t()) < 6e-3
    assert outbuf[:, :128].abs().sum().item() == 0 and outbuf[:, 512:].abs().sum().item() == 0


@pytest.mark.parametrize("group,k_skew,direct,split", [(1, 0, False, 1), (3, 0, False, 2), (-2, 0, False, 3), (16, 5, False, 0), (0, 0, True, 0)])
def test_gemm_pair_raster_and_epilogue_variants(C, group, k_skew, direct, split):
    # every raster / k-skew / epilogue choice of the CTA-pair kernel computes the same product, including on ragged edges
    torch.manual_seed(3)
    try:
        for (M, N, K) in [(1100, 1352, 520), (2048, 768, 1024)]:
            a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
            ref = a.float() @ b.float().t()
            st = _status()
            C.gemm_tuning(group, k_skew, direct, None, split)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            C.gemm(a, b, out, False, False, False, 1.0, st, 0, 2)
            assert _rel_err(out, ref) < 6e-3
            base = torch.randn(M, N, device="cuda", dtype=torch.float32)
            acc = base.clone()
            C.gemm(a, b, acc, False, False, True, 1.0, st, 0, 2)
            assert _rel_err(acc, base + ref) < 1e-5
            base16 = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
            acc16 = base16.clone()
            C.gemm(a, b, acc16, False, False, True, 1.0, st, 0, 2)
            assert _rel_err(acc16, base16.float() + ref) < 8e-3
            assert st.item() == 0
    finally:
        C.gemm_tuning(0, 0, False, None)


def test_gemm_pair_unaligned_output_takes_the_register_path(C):
    torch.manual_seed(4)
    M, N, K = 512, 300, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    buf = torch.zeros(M, N + 3, device="cuda", dtype=torch.bfloat16)  # row stride 303 elements: no tensor map possible
    out = buf[:, :N]
    st = _status()
    C.gemm(a, b, out, False, False, False, 1.0, st, 0, 2)
    assert st.item() == 0
    assert _rel_err(out, a.float() @ b.float().t()) < 6e-3
    assert buf[:, N:].abs().sum().item() == 0


@pytest.mark.parametrize("T,H,I", [(256, 256, 128), (1000, 512, 384), (4096, 1024, 2048)])
def test_gemm_with_swiglu_backward_epilogue(C, T, H, I):
    torch.manual_seed(7)
    dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(H, I, device="cuda", dtype=torch.bfloat16) * (H**-0.5)  # the down-projection weight [out, in]
    fc = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    dfc = torch.empty(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    act = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
    st = _status()
    C.gemm_swiglu_bwd(dy, w, fc, dfc, act, st)
    torch.cuda.synchronize()
    assert st.item() == 0
    # fp32 reference under autograd
    f32 = fc.float().requires_grad_(True)
    up, gate = f32[:, :I], f32[:, I:]
    y = up * torch.nn.functional.silu(gate)
    dact = dy.float() @ w.float()
    y.backward(dact)
    assert _rel_err(act, y) < 1e-2
    assert _rel_err(dfc, f32.grad) < 1e-2
    # same bits as the two-kernel path
    dact16 = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
    C.gemm(dy, w, dact16, False, True, False, 1.0, st, 0, 2)
    dfc2, act2 = C.swiglu_bwd(dact16, fc, True)
    assert torch.equal(dfc, dfc2) and torch.equal(act, act2)


def _with_canaries(rows, cols, dtype, pad=64):
    """A [rows, cols] view in the middle of a larger buffer filled with a canary value; returns (view, check)."""
    canary = 7.0
    buf = torch.full((rows + 2 * pad, cols + 2 * pad), canary, device="cuda", dtype=dtype)
    view = buf[pad : pad + rows, pad : pad + cols]

    def check():
        mask = torch.ones_like(buf, dtype=torch.bool)
        mask[pad : pad + rows, pad : pad + cols] = False
        assert bool((buf[mask] == canary).all()), "a kernel wrote outside of its output"

    return view, check


@pytest.mark.parametrize("shape", [(300, 520, 256), (1031, 264, 512)])
def test_bulk_store_epilogues_stay_inside_their_output(C, shape):
    """Outputs whose edges do not fall on tile boundaries, surrounded by canaries: the bulk tensor stores and reductions of
    the GEMM epilogues (bf16 store, fp32 accumulate, SwiGLU) and of the block-scaled GEMM must clip at the tensor's edge."""
    M, N, K = shape
    torch.manual_seed(6)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    st = _status()
    out, check = _with_canaries(M, N, torch.bfloat16)
    C.gemm(a, b, out, False, False, False, 1.0, st, 0, 2)
    check()
    assert _rel_err(out, a.float() @ b.float().t()) < 6e-3
    acc, check32 = _with_canaries(M, N, torch.float32)
    acc.zero_()
    C.gemm(a, b, acc, False, False, True, 1.0, st, 0, 2)
    check32()
    assert _rel_err(acc, a.float() @ b.float().t()) < 1e-5
    inter = 384
    w = torch.randn(2 * inter, K, device="cuda", dtype=torch.bfloat16) * K**-0.5
    fc, check_fc = _with_canaries(M, 2 * inter, torch.bfloat16)
    act, check_act = _with_canaries(M, inter, torch.bfloat16)
    C.gemm_swiglu(a, w, fc, act, st)
    check_fc()
    check_act()
    aq, asf = C.quantize_mx(a, False, 0)
    bq, bsf = C.quantize_mx(b, False, 0)
    mx, check_mx = _with_canaries(M, N, torch.bfloat16)
    C.gemm_mxfp8(aq, asf, bq, bsf, mx, False, False, 0, 0, False, 1.0, st)
    check_mx()
    torch.cuda.synchronize()
    assert st.item() == 0


@pytest.mark.parametrize("T,H,I", [(256, 256, 128), (1000, 512, 384), (4096, 1024, 2048)])
def test_gemm_with_swiglu_epilogue(C, T, H, I):
    torch.manual_seed(5)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(2 * I, H, device="cuda", dtype=torch.bfloat16) * (H**-0.5)
    fc = torch.empty(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    act = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
    st = _status()
    C.gemm_swiglu(x, w, fc, act, st)
    torch.cuda.synchronize()
    assert st.item() == 0
    ref_fc = x.float() @ w.float().t()
    assert _rel_err(fc, ref_fc) < 6e-3
    up, gate = ref_fc[:, :I], ref_fc[:, I:]
    assert _rel_err(act, up * torch.nn.functional.silu(gate)) < 1e-2
    # same bits as the two-kernel path: the activation is computed from the bf16-rounded projection
    fc2 = torch.empty_like(fc)
    C.gemm(x, w, fc2, False, False, False, 1.0, st, 0, 2)
    assert torch.equal(fc, fc2)
    assert torch.equal(act, C.swiglu_fwd(fc2))


@pytest.mark.parametrize("T,H", [(7, 64), (33, 4096), (5, 2560), (3, 8192), (2, 16384)])
def test_rmsnorm(C, T, H):
    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    y, rstd, h = C.rmsnorm_fwd(x, r, w, 1e-5, True)
    hf = (x.float() + r.float()).to(torch.bfloat16).float()
    assert torch.equal(h.float(), hf)
    ref = torch.nn.functional.rms_norm(hf, (H,), w.float(), 1e-5)
    assert _rel_err(y, ref) < 5e-3
    y2, rstd2 = C.rmsnorm_fwd(x, None, w, 1e-5, True)
    assert _rel_err(y2, torch.nn.functional.rms_norm(x.float(), (H,), w.float(), 1e-5)) < 5e-3
    # backward
    dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    dres = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    hh = hf.clone().requires_grad_(True)
    ww = w.float().clone().requires_grad_(True)
    torch.nn.functional.rms_norm(hh, (H,), ww, 1e-5).backward(dy.float())
    dw = torch.zeros(H, device="cuda")
    dh = C.rmsnorm_bwd(dy, h, w, rstd, dres, dw, False)
    assert _rel_err(dh, hh.grad + dres.float()) < 6e-3
    assert _rel_err(dw, ww.grad) < 2e-3
    C.rmsnorm_bwd(dy, h, w, rstd, None, dw, True)
    assert _rel_err(dw, 2 * ww.grad) < 2e-3


def test_swiglu(C):
    torch.manual_seed(0)
    x = torch.randn(37, 2 * 264, device="cuda", dtype=torch.bfloat16)
    xf = x.float().requires_grad_(True)
    up, gate = xf.chunk(2, dim=-1)
    ref = up * torch.nn.functional.silu(gate)
    y = C.swiglu_fwd(x)
    assert _rel_err(y, ref) < 5e-3
    dy = torch.randn_like(y)
    ref.backward(dy.float())
    dx, y2 = C.swiglu_bwd(dy, x, True)
    assert _rel_err(dx, xf.grad) < 6e-3
    assert torch.equal(y, y2)


@pytest.mark.parametrize("groups,qpg,d,rd", [(2, 4, 128, 128), (4, 1, 64, 64), (1, 8, 64, 32), (2, 1, 80, 80)])
def test_rope(C, groups, qpg, d, rd):
    torch.manual_seed(0)
    T = 19
    width = groups * (qpg + 2) * d
    qkv = torch.randn(T, width, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 50, (T,), device="cuda", dtype=torch.int32)
    inv = 1.0 / (10000 ** (torch.arange(0, rd, 2, device="cuda").float() / rd))
    ang = torch.arange(64, device="cuda").float()[:, None] * inv[None]
    cos_t, sin_t = ang.cos().contiguous(), ang.sin().contiguous()
    ref = qkv.float().view(T, groups, qpg + 2, d).clone()
    c = torch.cat([cos_t, cos_t], -1)[pos.long()][:, None, None, :]
    s = torch.cat([sin_t, sin_t], -1)[pos.long()][:, None, None, :]
    xr = ref[:, :, : qpg + 1, d - rd :]
    x1, x2 = xr.chunk(2, -1)
    ref[:, :, : qpg + 1, d - rd :] = xr * c + torch.cat([-x2, x1], -1) * s
    out = qkv.clone()
    C.rope_(out, cos_t, sin_t, pos, groups, qpg, d, rd, False)
    assert _rel_err(out, ref.view(T, width)) < 5e-3
    # the inverse rotation undoes it (up to bf16 rounding)
    C.rope_(out, cos_t, sin_t, pos, groups, qpg, d, rd, True)
    assert _rel_err(out, qkv) < 8e-3


def test_embedding(C):
    torch.manual_seed(0)
    w = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (4, 33), device="cuda")
    out = C.embedding_fwd(w, ids, 1.0)
    assert torch.equal(out, w[ids])
    dy = torch.randn(4, 33, 256, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(1000, 256, device="cuda")
    C.embedding_bwd(dy, ids, dw, 1.0)
    ref = torch.zeros_like(dw).index_add_(0, ids.flatten(), dy.float().view(-1, 256))
    assert _rel_err(dw, ref) < 1e-5


@pytest.mark.parametrize("V", [1000, 50264, 128256])
def test_cross_entropy(C, V):
    torch.manual_seed(0)
    T = 9
    logits = (3 * torch.randn(T, V, device="cuda")).to(torch.bfloat16)
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[3] = -100
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, labels, reduction="sum", ignore_index=-100)
    ref.backward()
    work = logits.clone()
    loss = C.cross_entropy_(work, labels, 1.0, 1.0, -100, True)
    assert abs(loss.sum().item() - ref.item()) / abs(ref.item()) < 2e-3
    assert _rel_err(work, lf.grad) < 8e-3
    assert work[3].abs().sum().item() == 0


def test_adamw_and_norm(C):
    torch.manual_seed(0)
    n = 4096 * 3 + 8
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-10, weight_decay=0.1)
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    total = torch.zeros(1, device="cuda")
    coef = torch.zeros(1, device="cuda")
    norm = torch.zeros(1, device="cuda")
    for step in range(1, 4):
        gg = g * step
        ref_p.grad = gg.clone()
        gn = torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        mine_g = gg.clone()
        C.sumsq(mine_g, total, False)
        C.clip_coef(total, 1.0, coef, norm)
        assert abs(norm.item() - gn.item()) / gn.item() < 1e-5
        C.adamw_step(p, m, v, mine_g, pb, 1e-2, 0.9, 0.95, 1e-10, 0.1, step, coef, 1.0, True)
        assert mine_g.abs().sum().item() == 0
        assert _rel_err(p, ref_p.data) < 1e-5
        assert torch.equal(pb, p.to(torch.bfloat16))


def test_casts(C):
    x = torch.randn(1003, device="cuda")
    y = torch.empty(1003, device="cuda", dtype=torch.bfloat16)
    C.cast_f32_to_bf16(x, y)
    assert torch.equal(y, x.to(torch.bfloat16))
    acc = torch.ones(1003, device="cuda")
    C.cast_bf16_to_f32(y, acc, True, 0.5)
    assert torch.allclose(acc, 1 + 0.5 * y.float())


def _attention_reference(qkv, cu, groups, qpg, d, scale, causal=True):
    """fp32 per-document softmax attention on the fused layout; returns (out, dqkv given dout) helpers."""
    T = qkv.shape[0]
    x = qkv.float().view(T, groups, qpg + 2, d)
    q = x[:, :, :qpg].reshape(T, groups * qpg, d)
    k = x[:, :, qpg].repeat_interleave(qpg, dim=1)
    v = x[:, :, qpg + 1].repeat_interleave(qpg, dim=1)
    outs = []
    bounds = cu.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        qi, ki, vi = (t[s:e].transpose(0, 1) for t in (q, k, v))
        att = (qi @ ki.transpose(1, 2)) * scale
        if causal:
            n = e - s
            att = att.masked_fill(torch.ones(n, n, device=att.device, dtype=torch.bool).triu(1), float("-inf"))
        outs.append((att.softmax(-1) @ vi).transpose(0, 1))
    return torch.cat(outs, 0).reshape(T, groups * qpg * d)


@pytest.mark.parametrize("groups,qpg,d", [(2, 4, 128), (3, 1, 64), (1, 2, 64), (2, 1, 128)])
@pytest.mark.parametrize("lengths", [[128], [300, 128, 77, 1000], [1, 2, 129, 255, 256, 257]])
def test_attention_fwd_bwd(C, groups, qpg, d, lengths):
    torch.manual_seed(0)
    T = sum(lengths)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device="cuda")
    width = groups * (qpg + 2) * d
    qkv = torch.randn(T, width, device="cuda", dtype=torch.bfloat16)
    scale = d**-0.5
    st = _status()
    out, lse = C.attn_fwd(qkv, cu, max(lengths), groups, qpg, d, scale, True, st)
    torch.cuda.synchronize()
    assert st.item() == 0
    q32 = qkv.float().requires_grad_(True)
    ref = _attention_reference(q32, cu, groups, qpg, d, scale)
    assert _rel_err(out, ref) < 1e-2
    assert _worst_row_err(out, ref) < 4e-2  # every token on its own, not only the tensor as a whole
    dout = torch.randn_like(out)
    ref.backward(dout.float())
    dqkv = C.attn_bwd(dout, qkv, out, lse, cu, max(lengths), groups, qpg, d, scale, True, st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert _worst_row_err(dqkv, q32.grad) < 6e-2
    g = q32.grad.view(T, groups, qpg + 2, d)
    mine = dqkv.float().view(T, groups, qpg + 2, d)
    assert _rel_err(mine[:, :, qpg + 1], g[:, :, qpg + 1]) < 2e-2  # dV
    assert _rel_err(mine[:, :, qpg], g[:, :, qpg]) < 2e-2  # dK
    assert _rel_err(mine[:, :, :qpg], g[:, :, :qpg]) < 2e-2  # dQ


@pytest.mark.parametrize("d,groups,qpg", [(80, 2, 2), (96, 1, 4), (32, 2, 1)])
def test_attention_head_widths_between_the_kernel_widths(C, d, groups, qpg):
    """Head widths the kernels do not have (80, 96, 32) run on the next wider kernel over zero-padded heads: outputs
    and gradients against the fp32 reference, with strict mode on so that a PyTorch path would raise."""
    from lm_engine import ops
    from lm_engine.ops.attention import attention_fused_qkv

    torch.manual_seed(0)
    lengths = [300, 77, 513]
    T = sum(lengths)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device="cuda")
    qkv = torch.randn(T, groups * (qpg + 2) * d, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    scale = d**-0.5
    ops.set_strict(True)
    try:
        out = attention_fused_qkv(qkv, cu, max(lengths), groups, qpg, d, scale, True)
        dout = torch.randn_like(out)
        out.backward(dout)
    finally:
        ops.set_strict(False)
    ops.check_status()
    q32 = qkv.detach().float().requires_grad_(True)
    ref = _attention_reference(q32, cu, groups, qpg, d, scale)
    ref.backward(dout.float())
    assert out.shape == ref.shape
    assert _rel_err(out, ref) < 1e-2
    assert _rel_err(qkv.grad, q32.grad) < 2e-2


@pytest.mark.parametrize("ranks,V", [(2, 1024), (4, 50264), (8, 128256)])
def test_vocabulary_parallel_cross_entropy_kernels(C, ranks, V):
    """Every rank's slice of the logits goes through the statistics kernel, the triples are combined as the
    tensor-parallel loss does, and every slice of the gradient comes from the gradient kernel: loss and gradient against
    fp32 cross entropy over the whole vocabulary."""
    from lm_engine.parallel.tensor_parallel import combine_shard_statistics

    torch.manual_seed(0)
    T = 257
    logits = (torch.randn(T, V, device="cuda") * 3).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    ref_in = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, labels, ignore_index=-100, reduction="none")
    row_scale = torch.rand(T, device="cuda") + 0.5
    ref.backward(row_scale)
    per = V // ranks
    shards = [logits[:, r * per : (r + 1) * per].contiguous() for r in range(ranks)]
    stats = torch.stack([C.ce_shard_stats(shards[r], labels, r * per, -100) for r in range(ranks)])
    lse, target = combine_shard_statistics(stats)
    loss = (lse - target) * (labels != -100)
    torch.testing.assert_close(loss, ref.detach(), atol=2e-4, rtol=1e-5)
    grad = torch.cat([C.ce_shard_grad(shards[r], labels, lse, row_scale, r * per, -100) for r in range(ranks)], dim=1)
    assert _rel_err(grad, ref_in.grad) < 5e-3
    assert grad[::7].abs().sum().item() == 0


def test_strict_mode_turns_a_pytorch_fallback_into_an_error(C):
    from lm_engine import ops

    a = torch.randn(64, 24, device="cuda", dtype=torch.bfloat16)[:, :20]  # row stride 24 elements is fine, inner size 20 is not
    w = torch.randn(32, 20, device="cuda", dtype=torch.bfloat16)
    before = sum(ops.fallback_counts().values())
    out = ops.linear(a, w)  # counted, logged once, computed by PyTorch
    assert _rel_err(out, a.float() @ w.float().t()) < 1e-2
    assert sum(ops.fallback_counts().values()) == before + 1
    ops.set_strict(True)
    try:
        with pytest.raises(RuntimeError, match="strict mode"):
            ops.linear(a, w)
    finally:
        ops.set_strict(False)


@pytest.mark.parametrize("T,H,I,E,k", [(300, 256, 128, 4, 2), (1000, 512, 256, 8, 4), (64, 128, 64, 40, 8)])
def test_scattered_experts_fwd_bwd(C, T, H, I, E, k):
    from lm_engine.ops.moe import scattered_experts_mlp

    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w_fc = (0.05 * torch.randn(E, 2 * I, H, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    w_proj = (0.05 * torch.randn(E, H, I, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    logits = torch.randn(T, E, device="cuda")
    top, experts = logits.topk(k, dim=-1)
    weights = top.softmax(-1).to(torch.bfloat16).requires_grad_(True)

    out = scattered_experts_mlp(x, w_fc, w_proj, weights, experts, E, k, "swiglu")
    dout = torch.randn_like(out)
    out.backward(dout)

    # fp32 reference: naive loop over experts
    xf, wf, wp, wr = (t.detach().float().requires_grad_(True) for t in (x, w_fc, w_proj, weights))
    ref = torch.zeros(T, H, device="cuda")
    for e in range(E):
        tok, slot = (experts == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok] @ wf[e].t()
        up, gate = h.chunk(2, -1)
        y = (up * torch.nn.functional.silu(gate)) @ wp[e].t()
        ref = ref.index_add(0, tok, y * wr[tok, slot].unsqueeze(-1))
    ref.backward(dout.float())
    assert _rel_err(out, ref) < 1.5e-2
    assert _rel_err(x.grad, xf.grad) < 2e-2
    assert _rel_err(w_fc.grad, wf.grad) < 2e-2
    assert _rel_err(w_proj.grad, wp.grad) < 2e-2
    assert _rel_err(weights.grad, wr.grad) < 3e-2


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim,groups,qpg", [(64, 2, 2), (128, 1, 4)])
def test_stickbreaking_attention_matches_dense_formulation(head_dim, groups, qpg):
    """Forward and backward kernels on a packed fused-qkv buffer against the fp32 dense formulation under autograd,
    document by document (outputs, remainders and the gradient of the fused buffer for random output / remainder gradients)."""
    from lm_engine import ops
    from lm_engine.hf_models.layers.stickbreaking import _FusedStickBreaking, stickbreaking_attention

    torch.manual_seed(0)
    lengths = [300, 1, 129, 514]
    bounds = [0]
    for n in lengths:
        bounds.append(bounds[-1] + n)
    T = bounds[-1]
    cu = torch.tensor(bounds, dtype=torch.int32, device="cuda")
    width = groups * (qpg + 2) * head_dim
    qkv = (torch.randn(T, width, device="cuda") * 0.7).bfloat16().requires_grad_(True)
    scale = head_dim**-0.5
    out, rem = _FusedStickBreaking.apply(qkv, cu, groups, qpg, head_dim, scale)
    ops.check_status()
    d_out = (torch.randn_like(out.float()) * 0.5).bfloat16()
    d_rem = torch.randn_like(rem) * 0.5
    torch.autograd.backward([out, rem], [d_out, d_rem])
    ops.check_status()
    got_grad = qkv.grad.float().clone()
    qkv.grad = None

    ref_in = qkv.detach().float().requires_grad_(True)
    ref_out, ref_rem = [], []
    for s, e in zip(bounds[:-1], bounds[1:]):
        v4 = ref_in[s:e].view(e - s, groups, qpg + 2, head_dim)
        q = v4[:, :, :qpg].reshape(e - s, groups * qpg, head_dim).transpose(0, 1)
        k = v4[:, :, qpg].repeat_interleave(qpg, dim=1).transpose(0, 1)
        v = v4[:, :, qpg + 1].repeat_interleave(qpg, dim=1).transpose(0, 1)
        o, r = stickbreaking_attention(q, k, v, scale)
        ref_out.append(o.transpose(0, 1).reshape(e - s, -1))
        ref_rem.append(r)
    ref_out, ref_rem = torch.cat(ref_out), torch.cat(ref_rem, dim=1)
    torch.testing.assert_close(out.float(), ref_out.detach(), atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(rem, ref_rem.detach(), atol=2e-2, rtol=2e-2)
    torch.autograd.backward([ref_out, ref_rem], [d_out.float(), d_rem])
    assert torch.isfinite(got_grad).all()
    assert _rel_err(got_grad, ref_in.grad) < 3e-2


@pytest.mark.gpu
@pytest.mark.parametrize("gru", [False, True])
@pytest.mark.parametrize("head_dim,clip", [(16, None), (64, 0.05), (128, None)])
def test_recurrent_scan_matches_the_step_by_step_loops(gru, head_dim, clip):
    """RNN / GRU scan kernels (forward, input / weight / initial-state gradients, clamped state gradient) against the
    PyTorch loops in fp32, over documents of different lengths."""
    from lm_engine.hf_models.layers.recurrent import gru_scan, rnn_scan
    from lm_engine.ops.recurrent import recurrent_scan

    torch.manual_seed(3)
    dev = torch.device("cuda")
    n, d, gates = 3, head_dim, (3 if gru else 1)
    lengths = [37, 5, 64]
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=dev)
    total = sum(lengths)
    x = (torch.randn(total, gates * n * d, device=dev) * 0.5).requires_grad_(True)
    w = (torch.randn(gates * n, d, d, device=dev) / d**0.5).requires_grad_(True)
    h0 = (torch.randn(len(lengths), n, d, device=dev) * 0.3).requires_grad_(True)
    dout = torch.randn(total, n, d, device=dev)

    out = recurrent_scan(x, w, cu, n, d, gru, clip, h0=h0)
    out.backward(dout)
    got = (out.detach().clone(), x.grad.clone(), w.grad.clone(), h0.grad.clone())
    x.grad = w.grad = h0.grad = None

    pieces = []
    start = 0
    for i, length in enumerate(lengths):
        xs = x[start:start + length].unsqueeze(0)
        state = h0[i:i + 1]
        if gru:
            xi, xf, xr = (t.reshape(1, length, n, d) for t in xs.chunk(3, dim=-1))
            wi, wf, wr = w.chunk(3, dim=0)
            pieces.append(gru_scan(xi, wi, xf, wf, xr, wr, state, clip).squeeze(0))
        else:
            pieces.append(rnn_scan(xs.reshape(1, length, n, d), w, state, clip).squeeze(0))
        start += length
    ref = torch.cat(pieces, dim=0)
    ref.backward(dout)
    for name, a, b in zip(("out", "dx", "dw", "dh0"), got, (ref.detach(), x.grad, w.grad, h0.grad)):
        err = (a - b).abs().max().item()
        scale = b.abs().max().item() + 1e-6
        assert err <= 2e-3 * scale + 1e-5, f"{name}: max abs error {err} against magnitude {scale}"


@pytest.mark.gpu
@pytest.mark.parametrize("entries,num_experts,first,local,capacity", [(5000, 40, 0, 40, None), (70001, 40, 10, 5, None),
                                                                   (9000, 8, 4, 4, 3000), (100, 256, 0, 256, None)])
def test_expert_layout_kernels_match_the_sort_based_layout(entries, num_experts, first, local, capacity):
    """The counting-sort kernels give, element for element, the stable argsort layout (also under a capacity bound)."""
    import lm_engine.ops.moe as moe

    torch.manual_seed(entries)
    experts = torch.randint(0, num_experts, (entries,), device="cuda", dtype=torch.int32)
    got = moe.build_grouped_layout(experts, num_experts, first_expert=first, num_local_experts=local, capacity_rows=capacity)
    assert got.dropped is not None
    available = moe.native_available
    moe.native_available = lambda: False  # the torch formulation of the same function
    try:
        ref = moe.build_grouped_layout(experts, num_experts, first_expert=first, num_local_experts=local, capacity_rows=capacity)
    finally:
        moe.native_available = available
    assert got.rows == ref.rows
    for name in ("dest_row", "src_entry", "tile_expert", "padded_offsets", "dropped"):
        assert torch.equal(getattr(got, name).cpu(), getattr(ref, name).cpu()), name
    if capacity is not None:
        assert int(got.dropped.item()) > 0


@pytest.mark.gpu
@pytest.mark.parametrize("w_mn", [False, True])
def test_dispatch_fused_into_the_grouped_gemm_matches_gather_then_gemm(w_mn):
    """Gather CTAs inside the grouped GEMM kernel (two source buffers standing in for two ranks) against the separate
    gather kernel followed by the grouped GEMM: identical gathered rows, identical products."""
    from lm_engine import ops
    from lm_engine.ops.moe import build_grouped_layout

    C = ops.native()
    st = ops.status_word(torch.device("cuda"))
    torch.manual_seed(5)
    tokens, hidden, inter, experts, k = 700, 512, 384, 6, 2
    bufs = [torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    selected = torch.randint(0, experts, (2 * tokens * k,), device="cuda", dtype=torch.int32)  # entries of both "ranks"
    layout = build_grouped_layout(selected, experts)
    w = torch.randn(experts, hidden, inter, device="cuda", dtype=torch.bfloat16) * 0.05 if w_mn else \
        torch.randn(experts, inter, hidden, device="cuda", dtype=torch.bfloat16) * 0.05
    ptrs = [b.data_ptr() for b in bufs]
    rows_ref = C.moe_gather(ptrs, [], layout.src_entry, hidden, tokens * k, k, bufs[0], layout.tile_expert, experts)
    out_ref = C.grouped_rows(rows_ref, w, layout.tile_expert, w_mn, st)
    for copy_ctas in (1, 7):
        rows, out = C.grouped_rows_dispatch(ptrs, layout.src_entry, tokens * k, k, w, layout.tile_expert, w_mn, st, copy_ctas)
        torch.cuda.synchronize()
        ops.check_status()
        used = int(layout.padded_offsets[-1].item())
        assert torch.equal(rows[:used], rows_ref[:used])
        assert torch.equal(out[:used], out_ref[:used])


@pytest.mark.gpu
@pytest.mark.parametrize("heads,groups,head_dim,state", [(4, 1, 64, 128), (6, 2, 32, 16), (2, 2, 64, 64)])
def test_ssd_scan_matches_the_chunked_formulation(heads, groups, head_dim, state):
    """The state-resident scan kernel against the chunked PyTorch formulation: outputs, final state and every gradient
    (x, a, b, c, initial state), with a gradient flowing into the final state as well."""
    from lm_engine.hf_models.layers.mamba2 import ssd_chunk_scan
    from lm_engine.ops.ssd import ssd_scan

    torch.manual_seed(1)
    dev = "cuda"
    B, L = 2, 150
    x = torch.randn(B, L, heads, head_dim, device=dev, requires_grad=True)
    a = (-torch.rand(B, L, heads, device=dev) * 0.5).requires_grad_(True)
    b = (torch.randn(B, L, groups, state, device=dev) * 0.3).requires_grad_(True)
    c = (torch.randn(B, L, groups, state, device=dev) * 0.3).requires_grad_(True)
    h0 = (torch.randn(B, heads, head_dim, state, device=dev) * 0.2).requires_grad_(True)
    dy = torch.randn(B, L, heads, head_dim, device=dev)
    dfinal = torch.randn(B, heads, head_dim, state, device=dev) * 0.1

    y, final = ssd_scan(x, a, b, c, h0)
    torch.autograd.backward([y, final], [dy, dfinal])
    got = [t.detach().clone() for t in (y, final, x.grad, a.grad, b.grad, c.grad, h0.grad)]
    for t in (x, a, b, c, h0):
        t.grad = None
    rep = heads // groups
    y_ref, final_ref = ssd_chunk_scan(x, a, b.repeat_interleave(rep, dim=2), c.repeat_interleave(rep, dim=2), 64, initial_state=h0)
    torch.autograd.backward([y_ref, final_ref], [dy, dfinal])
    ref = [y_ref.detach(), final_ref.detach(), x.grad, a.grad, b.grad, c.grad, h0.grad]
    for name, g, r in zip(("y", "final", "dx", "da", "db", "dc", "dh0"), got, ref):
        assert _rel_err(g, r) < 2e-4, (name, _rel_err(g, r))


@pytest.mark.parametrize("world,per_owner,capacity", [(2, 20, None), (4, 10, None), (8, 5, None), (4, 10, 0.5)])
def test_group_layout_equals_every_owners_own_layout(C, world, per_owner, capacity):
    """The layout a rank works out for the whole expert-parallel group from the shared routing table: its own part equals
    the single-rank layout bit for bit, and the (owner, row) it predicts for every entry is the row that owner's own
    layout gives the entry (-1 where the owner has to drop it)."""
    from lm_engine.ops.moe import build_group_layout, build_grouped_layout

    torch.manual_seed(7)
    num_experts = world * per_owner
    entries = 4096 * 8
    # skewed routing: some experts get far more than their share
    weights = torch.rand(num_experts, device="cuda") ** 3
    expert_of_entry = torch.multinomial(weights, entries, replacement=True).to(torch.int32)
    capacity_rows = None if capacity is None else int(capacity * entries / world)
    own = [build_grouped_layout(expert_of_entry, num_experts, first_expert=o * per_owner, num_local_experts=per_owner,
                                capacity_rows=capacity_rows) for o in range(world)]
    rows = own[0].rows
    owner_of_entry = (expert_of_entry // per_owner).long()
    expected = torch.stack([l.dest_row for l in own]).gather(0, owner_of_entry.unsqueeze(0)).squeeze(0)
    expected = torch.where(expected >= 0, owner_of_entry.to(torch.int32) * rows + expected, torch.full_like(expected, -1))
    for o in range(world):
        layout, global_row = build_group_layout(expert_of_entry, num_experts, per_owner, o, capacity_rows)
        assert layout.rows == rows
        assert torch.equal(layout.dest_row, own[o].dest_row)
        assert torch.equal(layout.src_entry, own[o].src_entry)
        assert torch.equal(layout.tile_expert, own[o].tile_expert)
        assert torch.equal(layout.padded_offsets, own[o].padded_offsets)
        assert torch.equal(layout.dropped, own[o].dropped)
        assert torch.equal(global_row, expected)
    if capacity is not None:
        assert int(sum(l.dropped for l in own).item()) > 0, "the capacity case is meant to drop entries"
