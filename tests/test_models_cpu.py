"""Model-level equivalences on CPU (the reference's single_gpu test ideas restated for this code base):
split/interleave of fused QKV is the identity, gated activations, padded == padding-free, full == incremental
decoding for every mixer type, cross-layer conversion is bit-equal, model variants train and generate."""

import pytest
import torch

from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM


def _attn(heads=4, kv=2, **extra):
    return dict(sequence_mixer_type="softmax_attention", num_attention_heads=heads, num_key_value_heads=kv, add_bias=False, **extra)


def _mlp(inter=64, **extra):
    return dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=inter, add_bias=False, **extra)


def _kw(layers=2, mixers=None, mlps=None, **extra):
    base = dict(vocab_size=128, hidden_size=32, num_layers=layers, position_embedding_type="rope", normalization_function="rmsnorm",
                tie_word_embeddings=False, sequence_mixer_blocks=mixers or [_attn()] * layers, mlp_blocks=mlps or [_mlp()] * layers)
    base.update(extra)
    return base


@pytest.mark.parametrize("heads,kv", [(4, 4), (4, 2), (4, 1)])
def test_split_interleave_roundtrip(heads, kv):
    from lm_engine.hf_models.layers.attention import (
        interleave_query_key_value_tensor_for_attention,
        split_query_key_value_tensor_for_attention,
    )

    d = 8
    q, k, v = torch.randn(heads * d, 32), torch.randn(kv * d, 32), torch.randn(kv * d, 32)
    fused = interleave_query_key_value_tensor_for_attention(q, k, v, heads, kv, d)
    q2, k2, v2 = split_query_key_value_tensor_for_attention(fused, heads, kv, d)
    assert torch.equal(q, q2) and torch.equal(k, k2) and torch.equal(v, v2)


def test_sigmoid_glu_matches_torch_glu():
    from lm_engine.hf_models.layers.activations import get_activation_function

    x = torch.randn(4, 16)
    up_gate = get_activation_function("sigmoid_glu")(x)
    assert torch.allclose(up_gate, torch.nn.functional.glu(x, dim=-1))
    assert torch.allclose(get_activation_function("glu")(x), torch.nn.functional.glu(x, dim=-1))


@pytest.mark.parametrize("pos", ["rope", "learned_absolute", "nope"])
@pytest.mark.parametrize("moe", [False, True])
def test_padded_equals_padding_free_and_masks(pos, moe):
    torch.manual_seed(0)
    mlps = [_mlp(), dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=32, add_bias=False, num_experts=4, num_experts_per_tok=2, shared_intermediate_size=16) if moe else _mlp()]
    config = GPTBaseConfig(**_kw(mlps=mlps, position_embedding_type=pos, max_position_embeddings=64))
    padded = GPTBaseForCausalLM(config).eval()
    packed = GPTBaseForCausalLM(config, use_padding_free_transformer=True).eval()
    packed.load_state_dict(padded.state_dict())
    docs = [torch.randint(3, 128, (10,)).tolist(), torch.randint(3, 128, (5,)).tolist()]
    # left-padded batch of the same two documents
    width = 10
    ids = torch.tensor([[0] * (width - len(d)) + d for d in docs])
    mask = torch.tensor([[0] * (width - len(d)) + [1] * len(d) for d in docs])
    # the first real token has no real context in the padded layout (it would be predicted from padding): mask it
    labels = torch.tensor([[-100] * (width - len(d) + 1) + d[1:] for d in docs])
    with torch.no_grad():
        a = padded(input_ids=ids, attention_mask=mask, labels=labels)
        b = packed(input_ids=docs, labels=docs)
    assert abs(a.loss.item() - b.loss.item()) < 1e-5
    assert torch.allclose(a.logits[0], b.logits[:10], atol=1e-5)
    assert torch.allclose(a.logits[1, 5:], b.logits[10:], atol=1e-5)
    # list inputs and explicit tensors + cu_seqlens agree exactly
    flat = torch.tensor(docs[0] + docs[1])
    with torch.no_grad():
        c = packed(input_ids=flat, cu_seqlens=torch.tensor([0, 10, 15], dtype=torch.int32), max_seqlen=10,
                   position_ids=torch.tensor(list(range(10)) + list(range(5))))
    assert torch.equal(b.logits, c.logits)
    with pytest.raises(ValueError):
        packed(input_ids=docs, attention_mask=mask)


def test_every_mixer_full_vs_incremental_vs_packed():
    torch.manual_seed(0)
    mixers = [
        _attn(),
        dict(sequence_mixer_type="stickbreaking_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False),
        dict(sequence_mixer_type="multihead_latent_attention", num_attention_heads=4, head_dim=16, query_compression_size=24, key_value_compression_size=16, add_bias=False),
        dict(sequence_mixer_type="mamba2", num_heads=8, state_size=16, num_groups=2, chunk_size=8, intermediate_size=64),
        dict(sequence_mixer_type="gru", state_size=32, num_heads=4, normalization_function="silu_gated_rmsnorm"),
        dict(sequence_mixer_type="rnn", state_size=32, num_heads=4, gradient_clipping=1.0),
        dict(sequence_mixer_type="causal_convolution", in_channels=48, out_channels=48, kernel_size=3, num_groups=4, activation_function="swiglu"),
    ]
    n = len(mixers)
    config = GPTBaseConfig(**_kw(layers=n, mixers=mixers, position_embedding_type="nope", tie_word_embeddings=True))
    model = GPTBaseForCausalLM(config).eval()
    ids = torch.randint(0, 128, (2, 12))
    with torch.no_grad():
        full = model(input_ids=ids).logits
        out = model(input_ids=ids[:, :8], use_cache=True)
        cache, steps = out.past_key_values, [out.logits]
        for t in range(8, 12):
            out = model(input_ids=ids[:, t : t + 1], past_key_values=cache, use_cache=True)
            steps.append(out.logits)
        assert torch.allclose(full, torch.cat(steps, 1), atol=1e-5)
        packed = GPTBaseForCausalLM(config, use_padding_free_transformer=True).eval()
        packed.load_state_dict(model.state_dict())
        assert torch.allclose(full.reshape(-1, 128), packed(input_ids=ids.tolist()).logits, atol=1e-5)
    model.train()
    model(input_ids=ids, labels=ids).loss.backward()


def test_stickbreaking_rows_sum_to_one():
    from lm_engine.hf_models.layers.stickbreaking import stickbreaking_attention

    q, k, v = torch.randn(2, 9, 8), torch.randn(2, 9, 8), torch.ones(2, 9, 8)
    out, rem = stickbreaking_attention(q, k, v, 0.3)
    # with v = 1 the output is the attention mass: mass + remainder = 1, first query sees nothing
    assert torch.allclose(out[..., 0] + rem, torch.ones(2, 9), atol=1e-5)
    assert torch.allclose(rem[:, 0], torch.ones(2))


def test_crosslayer_conversion_is_bit_equal_and_shares_kv():
    from lm_engine.hf_models import GPTCrossLayerForCausalLM, convert_gpt_base_to_gpt_crosslayer

    torch.manual_seed(0)
    base = GPTBaseForCausalLM(GPTBaseConfig(**_kw(layers=4))).eval()
    ids = torch.randint(0, 128, (2, 10))
    with torch.no_grad():
        ref = base(input_ids=ids, labels=ids)
        _, same = convert_gpt_base_to_gpt_crosslayer(base.config, base)
        out = same.eval()(input_ids=ids, labels=ids)
        assert torch.equal(out.logits, ref.logits) and torch.equal(out.loss, ref.loss)
        config, shared = convert_gpt_base_to_gpt_crosslayer(base.config, base, sharing_pattern=[0, 0, 2, 2])
        shared.eval()
        assert not any("kv_proj" in n for n, _ in shared.named_parameters() if ".h.1." in n or ".h.3." in n)
        packed = GPTCrossLayerForCausalLM(config, use_padding_free_transformer=True).eval()
        packed.load_state_dict(shared.state_dict())
        assert torch.allclose(packed(input_ids=ids.tolist()).logits, shared(input_ids=ids).logits.reshape(-1, 128), atol=1e-5)
        greedy = shared.generate(ids[:, :4], max_new_tokens=4)
        again = shared(input_ids=greedy[:, :-1]).logits.argmax(-1)
        assert torch.equal(again[:, 3:], greedy[:, 4:])


def test_model_variants_train_and_register():
    from transformers import AutoConfig, AutoModelForCausalLM

    ids = torch.randint(0, 128, (2, 10))
    for model_type in ("gpt_base", "palm", "ladder_residual", "gpt_crosslayer"):
        model = AutoModelForCausalLM.from_config(AutoConfig.for_model(model_type=model_type, **_kw()))
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        assert torch.isfinite(loss)
    desync = AutoModelForCausalLM.from_config(AutoConfig.for_model(
        model_type="desync_residual", pretraining_tensor_parallel_size=2,
        reduce_pattern=[{"attention": True, "mlp": False}] * 2, **_kw()))
    desync(input_ids=ids, labels=ids).loss.backward()


def test_desync_with_all_reduces_equals_gpt_base():
    from lm_engine.hf_models import DesyncResidualForCausalLM
    from lm_engine.hf_models.config import DesyncResidualConfig
    from lm_engine.hf_models.layers.attention import split_query_key_value_tensor_for_attention

    torch.manual_seed(0)
    kw = _kw(mixers=[_attn(4, 2)] * 2)
    base = GPTBaseForCausalLM(GPTBaseConfig(**kw)).eval()
    desync = DesyncResidualForCausalLM(DesyncResidualConfig(pretraining_tensor_parallel_size=2, **kw)).eval()
    sd = base.state_dict()
    new = {k: v for k, v in sd.items() if "sequence_mixer" not in k and "mlp_block" not in k}
    d = 8
    for i in range(2):
        p = f"transformer.h.{i}."
        q, k, v = split_query_key_value_tensor_for_attention(sd[p + "sequence_mixer.c_attn.weight"], 4, 2, d)
        # simulated rank r owns kv head r and its two query heads
        slices = [torch.cat([q[r * 2 * d : (r + 1) * 2 * d], k[r * d : (r + 1) * d], v[r * d : (r + 1) * d]]) for r in range(2)]
        new[p + "sequence_mixer.c_attn.weight"] = torch.stack(slices)
        new[p + "sequence_mixer.c_proj.weight"] = torch.stack(sd[p + "sequence_mixer.c_proj.weight"].chunk(2, dim=1))
        up, gate = sd[p + "mlp_block.c_fc.weight"].chunk(2, dim=0)
        new[p + "mlp_block.c_fc.weight"] = torch.stack([torch.cat([u, g]) for u, g in zip(up.chunk(2), gate.chunk(2))])
        new[p + "mlp_block.c_proj.weight"] = torch.stack(sd[p + "mlp_block.c_proj.weight"].chunk(2, dim=1))
    desync.load_state_dict(new)
    ids = torch.randint(0, 128, (2, 10))
    with torch.no_grad():
        assert torch.allclose(desync(input_ids=ids).logits, base(input_ids=ids).logits, atol=2e-5)


def test_greedy_generation_is_consistent_with_forward():
    torch.manual_seed(0)
    model = GPTBaseForCausalLM(GPTBaseConfig(**_kw())).eval()
    prompt = torch.randint(3, 128, (2, 5))
    out = model.generate(prompt, max_new_tokens=6, eos_token_id=-1)
    logits = model(input_ids=out[:, :-1]).logits
    assert torch.equal(logits.argmax(-1)[:, 4:], out[:, 5:])


def test_crosslayer_with_stickbreaking_layers():
    """Stick-breaking layers share keys / values across layers like softmax layers do: the conversion of a gpt_base model
    with stick-breaking mixers computes the same function, packed equals padded with sharing, greedy decoding with the
    cache repeats the full forward pass, and mixed sharing groups are refused."""
    from lm_engine.hf_models import GPTCrossLayerConfig, GPTCrossLayerForCausalLM, convert_gpt_base_to_gpt_crosslayer

    sb = dict(sequence_mixer_type="stickbreaking_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    torch.manual_seed(0)
    base = GPTBaseForCausalLM(GPTBaseConfig(**_kw(layers=4, mixers=[sb] * 4, position_embedding_type="nope"))).eval()
    with torch.no_grad():
        for name, p in base.named_parameters():
            if name.endswith("head_bias"):
                p.normal_(std=0.5)  # zero-initialised: make the remainder term visible
    ids = torch.randint(0, 128, (2, 12))
    with torch.no_grad():
        ref = base(input_ids=ids, labels=ids)
        _, same = convert_gpt_base_to_gpt_crosslayer(base.config, base)
        out = same.eval()(input_ids=ids, labels=ids)
        assert torch.allclose(out.logits, ref.logits, atol=1e-5) and torch.allclose(out.loss, ref.loss, atol=1e-6)
        config, shared = convert_gpt_base_to_gpt_crosslayer(base.config, base, sharing_pattern=[0, 0, 2, 2])
        shared.eval()
        packed = GPTCrossLayerForCausalLM(config, use_padding_free_transformer=True).eval()
        packed.load_state_dict(shared.state_dict())
        assert torch.allclose(packed(input_ids=ids.tolist()).logits, shared(input_ids=ids).logits.reshape(-1, 128), atol=1e-5)
        greedy = shared.generate(ids[:, :4], max_new_tokens=4)
        again = shared(input_ids=greedy[:, :-1]).logits.argmax(-1)
        assert torch.equal(again[:, 3:], greedy[:, 4:])
    # gradients reach the shared projection and the stick-breaking parameters
    shared.train()
    shared(input_ids=ids, labels=ids).loss.backward()
    grads = {n: p.grad for n, p in shared.named_parameters()}
    assert float(grads["transformer.h.0.kv_proj.kv_attn.weight"].abs().sum()) > 0
    assert float(grads["transformer.h.1.sequence_mixer.head_bias"].abs().sum()) > 0
    with pytest.raises(ValueError):
        GPTCrossLayerConfig(**_kw(layers=2, mixers=[_attn(), sb]), sharing_pattern=[0, 0])


def test_sliding_window_and_score_cap_of_the_attention_op():
    """The two flash-attention options of the reference's helper, evaluated by the PyTorch formulation: a window as wide as
    the document and a huge cap change nothing; a narrow window equals attention over the last keys only; the cap equals
    the explicit tanh formula."""
    from lm_engine.ops.attention import attention_fused_qkv, attention_varlen_reference

    torch.manual_seed(0)
    T, groups, qpg, d = 24, 2, 2, 8
    qkv = torch.randn(T, groups * (qpg + 2) * d)
    cu = torch.tensor([0, 10, 24], dtype=torch.int32)
    plain = attention_fused_qkv(qkv, cu, 14, groups, qpg, d)
    assert torch.allclose(attention_fused_qkv(qkv, cu, 14, groups, qpg, d, sliding_window=64, softcap=1e6), plain, atol=1e-5)
    windowed = attention_fused_qkv(qkv, cu, 14, groups, qpg, d, sliding_window=2)
    view = qkv.view(T, groups, qpg + 2, d)
    q, k, v = view[:, :, :qpg].reshape(T, groups * qpg, d), view[:, :, qpg], view[:, :, qpg + 1]
    for token, (lo, hi) in ((5, (3, 6)), (13, (11, 14)), (10, (10, 11))):  # the third one is the first token of its document
        for head in range(groups * qpg):
            scores = (k[lo:hi, head // qpg] @ q[token, head]) * d**-0.5
            expected = torch.softmax(scores, 0) @ v[lo:hi, head // qpg]
            assert torch.allclose(windowed.view(T, groups * qpg, d)[token, head], expected, atol=1e-5)
    capped = attention_varlen_reference(q, k, v, cu, None, True, 0.0, None, 0.5).view(T, groups * qpg, d)
    scores = (k[:4, 0] @ q[3, 0]) * d**-0.5
    assert torch.allclose(capped[3, 0], torch.softmax(0.5 * torch.tanh(scores / 0.5), 0) @ v[:4, 0], atol=1e-5)
