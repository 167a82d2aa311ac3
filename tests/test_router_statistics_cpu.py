"""The load-balancing loss of the MoE layers is finished once per forward pass from statistics the layers hand over; its
value and its gradients equal the per-layer formulation (softmax mass x token share per expert, plus the z loss)."""

import torch
import torch.nn.functional as F


def _per_layer(logits: torch.Tensor, selected: torch.Tensor, num_experts: int) -> torch.Tensor:
    probs = torch.softmax(logits, dim=-1)
    freq = torch.bincount(selected.flatten(), minlength=num_experts).float()
    balance = num_experts * (F.normalize(probs.sum(0), p=1, dim=0) * F.normalize(freq, p=1, dim=0)).sum()
    z = (torch.logsumexp(logits, dim=-1) ** 2).mean()
    return (balance + 0.1 * z).type_as(logits)


def test_deferred_router_statistics_equal_the_per_layer_losses():
    from lm_engine.hf_models.loss import add_aux_loss, add_router_statistics, clear_aux_loss, get_aux_loss

    torch.manual_seed(0)
    tokens, experts, top_k, layers = 96, 8, 2, 3
    logits = [torch.randn(tokens, experts, requires_grad=True) for _ in range(layers)]
    selected = [l.detach().topk(top_k, dim=-1).indices for l in logits]

    expected = sum(_per_layer(l, s, experts) for l, s in zip(logits, selected))
    expected_grads = torch.autograd.grad(expected, logits)

    clear_aux_loss()
    for l, s in zip(logits, selected):
        probs = torch.softmax(l, dim=-1)
        counts = torch.zeros(experts).index_add_(0, s.flatten(), torch.ones(s.numel()))
        add_router_statistics(probs.sum(0), counts, (torch.logsumexp(l, dim=-1) ** 2).mean(), l.dtype)
    add_aux_loss(0.25)  # a plain contribution from elsewhere keeps adding up as before
    total = get_aux_loss()
    assert torch.allclose(total, expected + 0.25, atol=1e-6)
    assert get_aux_loss() is total or torch.equal(get_aux_loss(), total)  # asking twice does not count the layers twice
    grads = torch.autograd.grad(total, logits)
    for g, e in zip(grads, expected_grads):
        assert torch.allclose(g, e, atol=1e-7)
    clear_aux_loss()
    assert get_aux_loss() == 0


def test_moe_layer_hands_over_statistics_only_while_training():
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM

    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    moe = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=32, num_experts=4, num_experts_per_tok=2, add_bias=False)
    config = GPTBaseConfig(vocab_size=64, hidden_size=32, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           tie_word_embeddings=False, sequence_mixer_blocks=[attn] * 2, mlp_blocks=[moe] * 2, router_aux_loss_coef=0.01)
    torch.manual_seed(1)
    model = GPTBaseForCausalLM(config)
    ids = torch.randint(0, 64, (2, 16))
    model.train()
    out = model(input_ids=ids, labels=ids)
    assert isinstance(out.aux_loss, torch.Tensor) and out.aux_loss.requires_grad and float(out.aux_loss) > 0
    out.loss.backward()
    gates = [p for n, p in model.named_parameters() if n.endswith("gate.weight")]
    assert gates and all(p.grad is not None and float(p.grad.abs().sum()) > 0 for p in gates)
    model.eval()
    with torch.no_grad():
        out = model(input_ids=ids, labels=ids)
    assert not isinstance(out.aux_loss, torch.Tensor) or float(out.aux_loss) == 0


def test_group_layout_without_the_kernel_is_the_owner_layout():
    from lm_engine.ops.moe import build_group_layout, build_grouped_layout

    torch.manual_seed(2)
    expert_of_entry = torch.randint(0, 8, (512,))
    layout, global_row = build_group_layout(expert_of_entry, 8, 4, 1, None)
    own = build_grouped_layout(expert_of_entry, 8, first_expert=4, num_local_experts=4)
    assert global_row is None  # the caller falls back to the exchange of row numbers
    assert layout.rows == own.rows and torch.equal(layout.dest_row, own.dest_row) and torch.equal(layout.src_entry, own.src_entry)
