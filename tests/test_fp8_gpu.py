"""fp8 GEMM and linear against dequantised fp32 references (GPU)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("fmt", [(0, 0), (1, 0)])
def test_fp8_gemm_layouts(a_mn, b_mn, fmt):
    from lm_engine import ops
    from lm_engine.fp8 import dequantize, quantize

    torch.manual_seed(0)
    C, st = ops.native(), ops.status_word(torch.device("cuda"))
    M, N, K = 384, 512, 640
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    aq, a_scale = quantize(a, fmt[0])
    bq, b_scale = quantize(b, fmt[1])
    a_ref, b_ref = dequantize(aq, a_scale, fmt[0]), dequantize(bq, b_scale, fmt[1])
    ref = (a_ref.t() if a_mn else a_ref) @ (b_ref if b_mn else b_ref.t())
    out = torch.empty(M, N, device="cuda", dtype=torch.float32)
    C.gemm_fp8(aq, bq, out, a_mn, b_mn, fmt[0], fmt[1], False, 1.0, a_scale, b_scale, st)
    ops.check_status()
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=1e-3)  # same inputs, fp32 accumulation: only summation order differs
    out_bf16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm_fp8(aq, bq, out_bf16, a_mn, b_mn, fmt[0], fmt[1], False, 1.0, a_scale, b_scale, st)
    torch.testing.assert_close(out_bf16.float(), ref, atol=0.3, rtol=2e-2)


def test_fp8_linear_forward_backward():
    from lm_engine.fp8 import fp8_linear

    torch.manual_seed(1)
    x = torch.randn(512, 768, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(1024, 768, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    bias = torch.randn(1024, device="cuda").bfloat16().requires_grad_(True)
    y = fp8_linear(x, w, bias)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, bias))
    ref = xr @ wr.t() + br
    ref.backward(dy.float())

    def relative(a, b):
        return float((a.float() - b).norm() / b.norm())

    assert relative(y, ref) < 0.05
    assert relative(x.grad, xr.grad) < 0.08
    assert relative(w.grad, wr.grad) < 0.08
    assert relative(bias.grad, br.grad) < 0.01


def test_fp8_manager_converts_linears():
    from lm_engine.fp8 import FP8Manager
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=256, add_bias=False)
    config = GPTBaseConfig(vocab_size=512, hidden_size=128, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           tie_word_embeddings=False, sequence_mixer_blocks=[attn] * 2, mlp_blocks=[mlp] * 2)
    torch.manual_seed(2)
    model = GPTBaseForCausalLM(config).cuda().bfloat16()
    ids = torch.randint(0, 512, (2, 64), device="cuda")
    reference = model(input_ids=ids, labels=ids).loss
    manager = FP8Manager([model])
    assert manager.converted == 8  # 4 linears per block, the LM head stays in bf16
    loss = model(input_ids=ids, labels=ids).loss
    loss.backward()
    assert abs(float(loss) - float(reference)) < 0.05 * float(reference)
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


@pytest.mark.parametrize("along_rows", [False, True])
@pytest.mark.parametrize("shape", [(256, 384), (1024, 128), (384, 1280)])
def test_mx_quantisation_kernel_matches_the_format_definition(along_rows, shape):
    """Payload bytes and scale codes of the kernel equal the PyTorch statement of OCP MXFP8 (e4m3, shared exponent
    floor(log2(amax)) - 8, round to nearest even), for blocks along the columns and along the rows."""
    from lm_engine import ops
    from lm_engine.fp8 import mx_quantize

    torch.manual_seed(0)
    C = ops.native()
    x = (torch.randn(*shape, device="cuda") * torch.exp(torch.randn(*shape, device="cuda") * 3)).bfloat16()
    x[0, :64] = 0  # an all-zero block
    q, sf = C.quantize_mx(x, along_rows, 0)
    ref_q, ref_s = mx_quantize(x, dim=0 if along_rows else 1)
    assert torch.equal(q, ref_q.view(torch.uint8))
    rows, k = (shape[1], shape[0]) if along_rows else shape
    plain = C.mx_scales_to_plain(sf, rows, k)
    expected = ref_s.t().contiguous() if along_rows else ref_s
    assert torch.equal(plain, expected)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(384, 512, 640), (128, 256, 128), (1000, 776, 1024)])
def test_block_scaled_gemm_against_the_dequantised_product(a_mn, b_mn, shape):
    from lm_engine import ops
    from lm_engine.fp8 import mx_dequantize, mx_quantize

    torch.manual_seed(1)
    C, st = ops.native(), ops.status_word(torch.device("cuda"))
    M, N, K = shape
    if (a_mn and M % 16) or (b_mn and N % 16):
        pytest.skip("MN-major 8-bit operands need a row length that is a multiple of 16 bytes")
    # values spread over many binades so that a wrong scale block shows up at once
    a = (torch.randn(M, K, device="cuda") * torch.exp2(torch.randint(-6, 6, (M, K // 32), device="cuda").repeat_interleave(32, 1).float())).bfloat16()
    b = (torch.randn(N, K, device="cuda") * torch.exp2(torch.randint(-6, 6, (N, K // 32), device="cuda").repeat_interleave(32, 1).float())).bfloat16()
    a_in = a.t().contiguous() if a_mn else a          # what the GEMM reads: [K, M] when MN-major
    b_in = b.t().contiguous() if b_mn else b
    aq, asf = C.quantize_mx(a_in, a_mn, 0)            # blocks always run along K
    bq, bsf = C.quantize_mx(b_in, b_mn, 0)
    a_ref = mx_dequantize(*mx_quantize(a, dim=1), dim=1)
    b_ref = mx_dequantize(*mx_quantize(b, dim=1), dim=1)
    ref = a_ref @ b_ref.t()
    out = torch.empty(M, N, device="cuda", dtype=torch.float32)
    C.gemm_mxfp8(aq, asf, bq, bsf, out, a_mn, b_mn, 0, 0, False, 1.0, st)
    ops.check_status()
    assert ((out - ref).norm() / ref.norm()).item() < 1e-5  # same operands, fp32 accumulation: only the summation order differs
    base = torch.randn(M, N, device="cuda")
    acc = base.clone()
    C.gemm_mxfp8(aq, asf, bq, bsf, acc, a_mn, b_mn, 0, 0, True, 0.5, st)
    assert ((acc - (base + 0.5 * ref)).norm() / ref.norm()).item() < 1e-5
    ops.check_status()


def test_mx_linear_runs_the_block_scaled_kernels_and_matches_the_emulation():
    from lm_engine import ops
    from lm_engine.fp8 import _MXLinear, mx_linear

    torch.manual_seed(2)
    x = torch.randn(512, 768, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(1024, 768, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    bias = torch.randn(1024, device="cuda").bfloat16().requires_grad_(True)
    ops.set_strict(True)
    try:
        y = mx_linear(x, w, bias)
        dy = torch.randn_like(y)
        y.backward(dy)
    finally:
        ops.set_strict(False)
    ops.check_status()
    xe, we, be = (t.detach().clone().requires_grad_(True) for t in (x, w, bias))
    ye = _MXLinear.apply(xe, we, be)
    ye.backward(dy)

    def relative(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm())

    assert relative(y, ye) < 1e-2          # same quantised operands; bf16 rounding of the emulation's operands and outputs
    assert relative(x.grad, xe.grad) < 1e-2
    assert relative(w.grad, we.grad) < 1e-2
    xr, wr = x.detach().float(), w.detach().float()
    assert relative(y, xr @ wr.t() + bias.detach().float()) < 0.05  # and close to the unquantised product


def test_mxfp8_training_follows_the_bf16_loss_curve():
    """50 optimizer steps of a small decoder on a fixed batch: the run whose linears use the MXFP8 kernels (forward, data
    gradient and weight gradient) stays within a few percent of the bf16 run at every step and ends as low."""
    from lm_engine import ops
    from lm_engine.fp8 import FP8Manager
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=512, add_bias=False)
    config = GPTBaseConfig(vocab_size=512, hidden_size=256, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           tie_word_embeddings=False, sequence_mixer_blocks=[attn] * 2, mlp_blocks=[mlp] * 2)
    torch.manual_seed(3)
    ids = torch.randint(0, 512, (4, 128), device="cuda")  # 512 tokens: every product's sizes are multiples of 128

    def curve(mx: bool) -> list[float]:
        torch.manual_seed(4)
        model = GPTBaseForCausalLM(config).cuda().bfloat16()
        if mx:
            manager = FP8Manager([model], recipe="mxfp8")
            assert manager.converted == 8
        optimizer = torch.optim.AdamW(model.parameters(), lr=2e-3, weight_decay=0.0)
        before = sum(ops.fallback_counts().values())
        losses = []
        for _ in range(50):
            loss = model(input_ids=ids, labels=ids).loss
            loss.backward()
            optimizer.step()
            optimizer.zero_grad(set_to_none=True)
            losses.append(float(loss))
        if mx:
            assert not any(key.startswith("mx_linear") for key in ops.fallback_counts()), "the MX linears left the block-scaled kernels"
        del before
        return losses

    bf16, mx = curve(False), curve(True)
    ops.check_status()
    assert bf16[-1] < 0.5 * bf16[0], "the task is expected to be learnable in 50 steps"
    for step, (a, b) in enumerate(zip(bf16, mx)):
        assert abs(a - b) < 0.08 * max(a, 0.2), (step, a, b)
