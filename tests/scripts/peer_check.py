"""Peer-memory collectives against NCCL on every visible GPU (launched with torchrun, one rank per GPU).

Checks, all with plain PyTorch references: barrier + reduce-scatter (multimem and plain peer loads), pull all-gather,
AdamW-with-broadcast against local AdamW + NCCL all-gather, and three training steps of a small bf16 model with the
engine on peer memory against the same run on NCCL. Prints ``PEER_CHECK_OK`` on rank 0 when everything matched.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from lm_engine import ops
from lm_engine.parallel.symmetric import PeerGroup


def check_collectives(rank: int, world: int, device: torch.device, multimem: bool) -> None:
    os.environ["LM_ENGINE_PEER_MULTIMEM"] = "1" if multimem else "0"
    peer = PeerGroup(None, device)
    C = ops.native()
    n = 1 << 22  # per-rank shard elements
    torch.manual_seed(100 + rank)

    # reduce-scatter of fp32
    buf = peer.alloc(n * world, torch.float32)
    buf.tensor.copy_(torch.randn(n * world, device=device))
    expected = torch.empty(n, device=device)
    dist.reduce_scatter_tensor(expected, buf.tensor.clone(), op=dist.ReduceOp.SUM)
    out = torch.empty(n, device=device)
    peer.barrier()
    peer.reduce_scatter_f32(buf, buf.tensor[rank * n : (rank + 1) * n], out)
    peer.barrier()
    peer.check()
    torch.testing.assert_close(out, expected, atol=1e-5, rtol=1e-5)
    # in place (the engine's use)
    peer.reduce_scatter_f32(buf, buf.tensor[rank * n : (rank + 1) * n], buf.tensor[rank * n : (rank + 1) * n])
    peer.barrier()
    torch.testing.assert_close(buf.tensor[rank * n : (rank + 1) * n], expected, atol=1e-5, rtol=1e-5)

    # pull all-gather of bf16
    gathered = peer.alloc(n * world, torch.bfloat16)
    mine = torch.randn(n, device=device).bfloat16()
    gathered.tensor[rank * n : (rank + 1) * n].copy_(mine)
    reference = torch.empty(n * world, device=device, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(reference, mine)
    peer.barrier()
    peer.all_gather(gathered, gathered.tensor, n)
    peer.barrier()
    peer.check()
    assert torch.equal(gathered.tensor, reference)

    # AdamW whose bf16 result lands on every rank
    p = torch.randn(n, device=device)
    g = torch.randn(n, device=device)
    m = torch.rand(n, device=device) * 0.1
    v = torch.rand(n, device=device) * 0.1
    p2, g2, m2, v2 = p.clone(), g.clone(), m.clone(), v.clone()
    scale = torch.full((1,), 0.5, device=device)
    local_bf16 = torch.empty(n, device=device, dtype=torch.bfloat16)
    C.adamw_step(p2, m2, v2, g2, local_bf16, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, scale, 0.25, True)
    dist.all_gather_into_tensor(reference, local_bf16)
    target = peer.alloc(n * world, torch.bfloat16)
    peer.barrier()
    C.adamw_step_bcast(p, m, v, g, target.ptrs, target.multicast_ptr, rank * n, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, scale, 0.25, True)
    peer.barrier()
    peer.check()
    assert torch.equal(p, p2) and torch.equal(m, m2) and torch.equal(v, v2) and float(g.abs().max()) == 0.0
    assert torch.equal(target.tensor, reference)
    if rank == 0:
        print(f"collectives ok (multimem={multimem}, multicast address {'present' if buf.multicast_ptr else 'absent'})", flush=True)


def train_losses(fused: bool, steps: int = 3, resident: bool = True) -> list[float]:
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM
    from lm_engine.optimization.optimizer import FusedAdamW
    from lm_engine.parallel.engine import ShardedTrainingEngine

    device = torch.device("cuda", torch.cuda.current_device())
    layer_attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    layer_mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=512, add_bias=False)
    config = GPTBaseConfig(vocab_size=1024, hidden_size=256, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           max_position_embeddings=256, tie_word_embeddings=False, sequence_mixer_blocks=[layer_attn] * 2, mlp_blocks=[layer_mlp] * 2)
    torch.manual_seed(7)
    model = GPTBaseForCausalLM(config)
    engine = ShardedTrainingEngine(model, compute_dtype=torch.bfloat16, device=device, fused_collectives=fused, resident_parameters=resident)
    assert (engine.peer is not None) == fused, "peer memory was not set up"
    if not resident:
        assert all(not u.resident for u in engine.units if u.module is not None), "blocks are expected to be sharded"
    optimizer = FusedAdamW([seg.master for seg in engine.segments()], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    rank = dist.get_rank()
    losses = []
    for step in range(steps):
        torch.manual_seed(1000 + 10 * step + rank)
        ids = torch.randint(0, 1024, (4, 256), device=device)
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        engine.fold_autograd_grads()
        engine.optimizer_step(optimizer, None, max_norm=1.0)
        value = loss.detach().float()
        dist.all_reduce(value)
        losses.append(float(value))
    if engine.peer is not None:
        engine.peer.check()
    checksum = 0.0
    for unit in engine.units:  # sum over the whole compute copy, whichever way it is stored
        part = unit.compute_shard.float().sum()
        if unit.world > 1:
            dist.all_reduce(part)
        checksum += float(part)
    return losses + [checksum]


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    device = torch.device("cuda", torch.cuda.current_device())
    from lm_engine.utils import init_distributed

    init_distributed()
    for multimem in (False, True):
        check_collectives(rank, world, device, multimem)
    os.environ["LM_ENGINE_PEER_MULTIMEM"] = "1"
    nccl = train_losses(False)
    peer = train_losses(True)
    sharded = train_losses(False, resident=False)  # blocks gathered and released one by one (NCCL collectives)
    if rank == 0:
        print("nccl", nccl, "\npeer", peer, "\nsharded parameters", sharded, flush=True)
    for a, b, c in zip(nccl, peer, sharded):
        assert abs(a - b) <= 2e-3 * max(1.0, abs(a)), (nccl, peer)
        assert abs(a - c) <= 2e-3 * max(1.0, abs(a)), (nccl, sharded)
    dist.barrier()
    if rank == 0:
        print("PEER_CHECK_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
