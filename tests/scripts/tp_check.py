"""Tensor-parallel model against the single-device model, on CPU with gloo (launched with torchrun, world = tp size).

For several configurations: the TP model built with the same seed holds exactly the slices of the single-device
weights; logits, loss and (after the partial-gradient reduction) gradients agree; shard -> unshard round-trips; the
plain-concatenation fixer agrees with the unsharder. Prints ``TP_CHECK_OK`` on rank 0.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM
from lm_engine.hf_models.models.tensor_parallel import GPTBaseForCausalLM_TP, LadderResidualForCausalLM_TP, reduce_tensor_parallel_grads
from lm_engine.hf_models.tp_weights import fix_unsharded_state_dict, shard_state_dict, unshard_tensor_parallel_state_dicts
from lm_engine.utils import ProcessGroupManager, init_distributed


def make_config(kind: str, cls=GPTBaseConfig):
    heads = dict(mha=(4, 4), gqa=(8, 4), mqa=(4, 1))[kind.split("-")[0]]
    bias = "bias" in kind
    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=heads[0], num_key_value_heads=heads[1], add_bias=bias)
    dense = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=96, add_bias=bias)
    moe = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=32, add_bias=False, num_experts=4, num_experts_per_tok=2,
               shared_intermediate_size=48 if "shared" in kind else None)
    gelu = dict(mlp_type="MLP", activation_function="gelu_pytorch_tanh", intermediate_size=96, add_bias=bias)
    mlps = [dense, moe] if "moe" in kind else [dense, gelu]
    position = "learned_absolute" if "wpe" in kind else "rope"
    return cls(vocab_size=250, hidden_size=64, num_layers=2, max_position_embeddings=64, position_embedding_type=position,
               normalization_function="layernorm" if bias else "rmsnorm", tie_word_embeddings="tied" in kind, router_aux_loss_coef=0.01,
               sequence_mixer_blocks=[attn, attn], mlp_blocks=mlps, m_width=2.0 if "mup" in kind else None)


def close(a, b, what, atol=2e-5):
    if not torch.allclose(a, b, atol=atol, rtol=1e-4):
        raise AssertionError(f"{what}: max abs diff {(a - b).abs().max().item():.3e}")


def check(kind: str, sequence_parallel: bool, packed: bool) -> None:
    rank, world = dist.get_rank(), dist.get_world_size()
    config = make_config(kind)
    torch.manual_seed(1234)
    full = GPTBaseForCausalLM(config, use_padding_free_transformer=packed)
    torch.manual_seed(1234)
    local = GPTBaseForCausalLM_TP(config, use_padding_free_transformer=packed, sequence_parallel=sequence_parallel)
    full_state = full.state_dict()

    # same seed -> the local model holds the slices of the single-device model
    expected_local = shard_state_dict(config, full_state, rank, world)
    local_state = local.state_dict()
    assert set(expected_local) == set(local_state), (sorted(set(expected_local) ^ set(local_state)))
    for key, value in expected_local.items():
        assert torch.equal(local_state[key], value), f"{kind}: initial value of {key} is not the slice of the full model"

    # unshard (gather every rank's state dict) and the concatenation fixer
    gathered = [None] * world
    dist.all_gather_object(gathered, {k: v.clone() for k, v in local_state.items()})
    unsharded = unshard_tensor_parallel_state_dicts(config, gathered)
    assert set(unsharded) == set(full_state)
    for key, value in full_state.items():
        assert torch.equal(unsharded[key], value), f"{kind}: unsharded {key} differs"
    naive = {}
    for key in local_state:
        pieces = [g[key] for g in gathered]
        dim = getattr(dict(local.named_parameters())[key], "_tp_shard_dim", None)
        naive[key] = pieces[0] if dim is None else torch.cat(pieces, dim=dim)
    fixed = fix_unsharded_state_dict(config, naive, world)
    for key, value in full_state.items():
        assert torch.equal(fixed[key], value), f"{kind}: fixed {key} differs"

    # forward / backward parity
    torch.manual_seed(99)
    if packed:
        lengths = [24, 40]
        ids = torch.randint(0, 250, (sum(lengths),))
        cu = torch.tensor([0, 24, 64], dtype=torch.int32)
        pos = torch.cat([torch.arange(n) for n in lengths])
        inputs = dict(input_ids=ids, labels=ids.clone(), cu_seqlens=cu, max_seqlen=40, position_ids=pos)
    else:
        ids = torch.randint(0, 250, (2, 32))
        inputs = dict(input_ids=ids, labels=ids.clone())
    full.train()
    local.train()
    ref = full(**inputs)
    out = local(**inputs)
    close(out.logits, ref.logits, f"{kind} sp={sequence_parallel} packed={packed} logits")
    close(out.loss, ref.loss, f"{kind} loss", atol=1e-5)
    sliced = local(**inputs, output_parallel_lm_logits=True)
    assert sliced.logits.shape[-1] == local.get_output_embeddings().weight.shape[0]
    ref.loss.backward()
    out.loss.backward()
    reduce_tensor_parallel_grads(local, sequence_parallel)
    full_grads = {k: p.grad for k, p in full.named_parameters()}
    expected = shard_state_dict(config, full_grads, rank, world)
    for key, p in local.named_parameters():
        close(p.grad, expected[key], f"{kind} sp={sequence_parallel} packed={packed} grad of {key}", atol=5e-5)


def check_ladder() -> None:
    from lm_engine.hf_models import LadderResidualConfig, LadderResidualForCausalLM

    config = make_config("gqa", LadderResidualConfig)
    torch.manual_seed(5)
    full = LadderResidualForCausalLM(config)
    torch.manual_seed(5)
    local = LadderResidualForCausalLM_TP(config, sequence_parallel=True)
    ids = torch.randint(0, 250, (2, 32))
    close(local(input_ids=ids).logits, full(input_ids=ids).logits, "ladder logits")

    # overlapped layer: the row-parallel reductions are only started inside the sub-block and waited for one sub-block
    # later; outputs and gradients must not change (with and without sequence parallelism, padded and packed)
    from lm_engine.enums import Kernel
    from lm_engine.kernels import enable_kernels

    for sequence_parallel in (False, True):
        for packed in (False, True):
            torch.manual_seed(5)
            model = LadderResidualForCausalLM_TP(config, sequence_parallel=sequence_parallel, use_padding_free_transformer=packed)
            model.train()
            batch = [row.tolist() for row in ids] if packed else ids
            plain = model(input_ids=batch, labels=batch)
            plain.loss.backward()
            plain_grads = {k: p.grad.clone() for k, p in model.named_parameters()}
            model.zero_grad()
            with enable_kernels([Kernel.ladder_residual_overlapped_layer]):
                overlapped = model(input_ids=batch, labels=batch)
                assert model.transformer.h["0"].sequence_mixer.c_proj.overlap_reduction, "the overlapped layer did not switch on"
                overlapped.loss.backward()
            close(overlapped.loss, plain.loss, f"ladder overlapped loss sp={sequence_parallel} packed={packed}")
            for key, p in model.named_parameters():
                close(p.grad, plain_grads[key], f"ladder overlapped grad of {key} sp={sequence_parallel} packed={packed}", atol=5e-6)


def check_pipeline_stages() -> None:
    """Two stages chained by hand reproduce the single-stage model."""
    config = make_config("gqa-moe")
    torch.manual_seed(77)
    whole = GPTBaseForCausalLM_TP(config, sequence_parallel=True)
    state = whole.state_dict()
    stages = [GPTBaseForCausalLM_TP(config, sequence_parallel=True, num_pipeline_stages=2, pipeline_stage_id=s) for s in range(2)]
    for stage in stages:
        own = stage.state_dict()
        assert set(own) <= set(state)
        stage.load_state_dict({k: state[k] for k in own})
    assert set(stages[0].state_dict()) | set(stages[1].state_dict()) == set(state)
    ids = torch.randint(0, 250, (2, 32))
    for m in [whole] + stages:
        m.train()
    ref = whole(input_ids=ids, labels=ids)
    hidden, aux = stages[0](input_ids=ids)
    out = stages[1](pipeline_parallel_input=(hidden, aux), labels=ids)
    close(out.logits, ref.logits, "pipeline logits")
    close(out.loss, ref.loss, "pipeline loss")


def main() -> None:
    world = int(os.environ["WORLD_SIZE"])
    init_distributed(tensor_parallel_world_size=world)
    assert ProcessGroupManager.get_tensor_parallel_world_size() == world
    for kind in ("mha", "gqa-bias-wpe", "mqa", "mqa-bias", "gqa-moe", "gqa-moe-shared", "gqa-tied-mup"):
        for sequence_parallel in (False, True):
            for packed in (False, True):
                if packed and "wpe" in kind:
                    continue
                check(kind, sequence_parallel, packed)
        if dist.get_rank() == 0:
            print(f"{kind} ok", flush=True)
    check_ladder()
    check_pipeline_stages()
    dist.barrier()
    if dist.get_rank() == 0:
        print("TP_CHECK_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
