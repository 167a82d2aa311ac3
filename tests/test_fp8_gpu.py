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
