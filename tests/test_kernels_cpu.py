"""CPU statements of device-side algorithms: the expert row layout, the MX block format and the SSD scan function
(the kernels themselves are tested on a GPU in test_kernels_gpu.py)."""


def test_grouped_layout_capacity_bound_drops_the_overflow_and_counts_it():
    """Rows past the capacity bound are dropped (dest_row -1), counted, and the expert ranges are clipped to the buffer."""
    import torch

    from lm_engine.ops.moe import TILE, build_grouped_layout

    torch.manual_seed(0)
    experts = torch.randint(0, 8, (9000,), dtype=torch.int32)
    free = build_grouped_layout(experts, 8, first_expert=4, num_local_experts=4)
    assert int(free.dropped.item()) == 0 and (free.dest_row >= 0).sum().item() == ((experts >= 4).sum().item())
    bound = build_grouped_layout(experts, 8, first_expert=4, num_local_experts=4, capacity_rows=3000)
    assert bound.rows == 3072 and bound.rows % TILE == 0
    placed = int((bound.dest_row >= 0).sum().item())
    assert placed + int(bound.dropped.item()) == int((experts >= 4).sum().item()) and int(bound.dropped.item()) > 0
    assert int(bound.dest_row.max().item()) < bound.rows and int(bound.padded_offsets[-1].item()) <= bound.rows
    # every placed entry is found again through src_entry, and the kept prefix matches the unbounded layout
    rows = bound.dest_row[bound.dest_row >= 0].long()
    assert torch.equal(bound.src_entry[rows].long(), torch.nonzero(bound.dest_row >= 0).flatten())
    keep = bound.dest_row >= 0
    assert torch.equal(bound.dest_row[keep], free.dest_row[keep])


def test_mx_quantisation_follows_the_block_format():
    """One power-of-two scale per 32 elements, e4m3 payload: exact for values that e4m3 holds after the shift, relative
    error below 2^-3 otherwise, saturation at the block maximum, and quantisation along any dimension."""
    import torch

    from lm_engine.fp8 import MX_BLOCK, mx_dequantize, mx_quantize

    torch.manual_seed(0)
    x = torch.randn(6, 128) * torch.logspace(-6, 6, 6).unsqueeze(1)
    payload, scales = mx_quantize(x)
    assert payload.dtype == torch.float8_e4m3fn and payload.shape == x.shape
    assert scales.dtype == torch.uint8 and scales.shape == (6, 128 // MX_BLOCK)
    back = mx_dequantize(payload, scales)
    blocks, back_blocks = x.view(6, 4, MX_BLOCK), back.view(6, 4, MX_BLOCK)
    amax = blocks.abs().amax(-1, keepdim=True)
    # elements well above the block's underflow level keep 3 mantissa bits (relative error at most 2^-4); the block
    # maximum may saturate from just below 512 to 448, which is the worst case 2^-3
    big = blocks.abs() > amax * 2.0**-6
    assert ((back_blocks - blocks).abs()[big] <= blocks.abs()[big] * 2.0**-3 + 1e-30).all()
    inside = big & (blocks.abs() * torch.exp2(127.0 - scales.float()).unsqueeze(-1) <= 448)
    assert ((back_blocks - blocks).abs()[inside] <= blocks.abs()[inside] * 2.0**-4 + 1e-30).all()
    # the scale is the power of two that puts the block maximum into [256, 512) before saturation at 448
    shifted = amax.squeeze(-1) * torch.exp2(127.0 - scales.float())
    assert ((shifted >= 256 * (1 - 1e-6)) & (shifted < 512)).all()
    # powers of two survive exactly, and quantising along dim 0 equals quantising the transpose along dim 1
    exact = torch.tensor([[2.0 ** (k % 15) for k in range(32)]])  # 2^0 .. 2^14: within e4m3's normal range after the shift
    assert torch.equal(mx_dequantize(*mx_quantize(exact)), exact)
    y = torch.randn(64, 8)
    p0, s0 = mx_quantize(y, dim=0)
    p1, s1 = mx_quantize(y.t().contiguous(), dim=1)
    assert torch.equal(p0.float(), p1.float().t()) and torch.equal(s0, s1.t())


def test_mx_linear_gradients_track_the_unquantised_layer():
    import torch

    from lm_engine.fp8 import mx_linear

    torch.manual_seed(1)
    x = torch.randn(64, 96, requires_grad=True)
    w = (torch.randn(128, 96) * 0.1).requires_grad_(True)
    b = torch.zeros(128, requires_grad=True)
    dy = torch.randn(64, 128)
    mx_linear(x, w, b).backward(dy)
    got = [t.grad.clone() for t in (x, w, b)]
    for t in (x, w, b):
        t.grad = None
    torch.nn.functional.linear(x, w, b).backward(dy)
    for g, t in zip(got, (x, w, b)):
        rel = (g - t.grad).norm() / t.grad.norm()
        assert rel < 0.06, rel
    assert torch.equal(got[2], b.grad)


def test_mxfp8_recipe_converts_the_linears_of_a_model():
    """``FP8Manager(recipe="mxfp8")`` switches the block linears (not the LM head) to MX operands; the loss stays close to
    the unquantised model and every parameter still receives a gradient."""
    import torch

    from lm_engine.fp8 import FP8Manager
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    torch.manual_seed(0)
    config = GPTBaseConfig(
        vocab_size=128, hidden_size=64, num_layers=2, max_position_embeddings=64, position_embedding_type="rope",
        normalization_function="rmsnorm", tie_word_embeddings=False,
        sequence_mixer_blocks=[dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)] * 2,
        mlp_blocks=[dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=128, add_bias=False)] * 2,
    )
    model = GPTBaseForCausalLM(config)
    ids = torch.randint(0, 128, (2, 32))
    reference = float(model(input_ids=ids, labels=ids).loss)
    manager = FP8Manager([model], recipe="mxfp8")
    assert manager.converted == 8  # c_attn, c_proj, c_fc, c_proj of two blocks
    out = model(input_ids=ids, labels=ids)
    assert abs(float(out.loss) - reference) < 0.05 * reference
    out.loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


def test_ssd_scan_function_on_cpu_matches_the_chunked_formulation_packed_and_batched():
    """The autograd function around the scan (step-by-step recurrence on CPU): batched rows with an initial state and a
    gradient into the final state, and packed documents whose state restarts at every document."""
    import torch

    from lm_engine.hf_models.layers.mamba2 import ssd_chunk_scan
    from lm_engine.ops.ssd import ssd_scan

    torch.manual_seed(2)
    H, G, P, N = 4, 2, 8, 16

    def inputs(B, L):
        x = torch.randn(B, L, H, P, requires_grad=True)
        a = (-torch.rand(B, L, H) * 0.5).requires_grad_(True)
        b = (torch.randn(B, L, G, N) * 0.3).requires_grad_(True)
        c = (torch.randn(B, L, G, N) * 0.3).requires_grad_(True)
        return x, a, b, c

    def chunked(x, a, b, c, h0=None):
        return ssd_chunk_scan(x, a, b.repeat_interleave(H // G, dim=2), c.repeat_interleave(H // G, dim=2), 16, initial_state=h0)

    def grads(tensors):
        out = [t.grad.clone() for t in tensors]
        for t in tensors:
            t.grad = None
        return out

    # batched, with initial state and final-state gradient
    x, a, b, c = inputs(2, 40)
    h0 = (torch.randn(2, H, P, N) * 0.2).requires_grad_(True)
    dy, dfinal = torch.randn(2, 40, H, P), torch.randn(2, H, P, N) * 0.1
    y, final = ssd_scan(x, a, b, c, h0)
    torch.autograd.backward([y, final], [dy, dfinal])
    got = [y.detach(), final.detach()] + grads([x, a, b, c, h0])
    y_ref, final_ref = chunked(x, a, b, c, h0)
    torch.autograd.backward([y_ref, final_ref], [dy, dfinal])
    ref = [y_ref.detach(), final_ref.detach()] + grads([x, a, b, c, h0])
    for g, r in zip(got, ref):
        assert (g - r).norm() <= 1e-4 * r.norm() + 1e-6

    # packed: three documents (one of a single token) in one row
    lengths = [13, 1, 26]
    cu = torch.tensor([0, 13, 14, 40], dtype=torch.int32)
    x, a, b, c = inputs(1, 40)
    dy = torch.randn(1, 40, H, P)
    y, _ = ssd_scan(x, a, b, c, cu_seqlens=cu)
    y.backward(dy)
    got = [y.detach()] + grads([x, a, b, c])
    pieces, start = [], 0
    for n in lengths:
        sl = slice(start, start + n)
        pieces.append(chunked(x[:, sl], a[:, sl], b[:, sl], c[:, sl])[0])
        start += n
    y_ref = torch.cat(pieces, dim=1)
    y_ref.backward(dy)
    ref = [y_ref.detach()] + grads([x, a, b, c])
    # the decay of a document's first token multiplies a zero state: its gradient is zero in both formulations
    for name, g, r in zip(("y", "dx", "da", "db", "dc"), got, ref):
        assert (g - r).norm() <= 1e-4 * r.norm() + 1e-6, name
