"""Hybrid sharding (replicate x shard) on GPUs: 4 ranks as 2 replicas of 2 shards, launched with torchrun.

Three training steps of a small bf16 model with the engine on the hybrid topology, gradients reduce-scattered inside
each shard group (peer-memory kernels or NCCL) and all-reduced across the replicas, against the same run on plain
4-way sharding: the same global batch must give the same losses. Prints ``HSDP_CHECK_OK`` on rank 0.
"""

import json
import os
import subprocess
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def losses(replicas: int, shards: int, fused: bool) -> list[float]:
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM
    from lm_engine.optimization.optimizer import FusedAdamW
    from lm_engine.parallel.engine import ShardedTrainingEngine
    from lm_engine.utils import ProcessGroupManager, init_distributed

    init_distributed(data_parallel_replication_world_size=replicas, data_parallel_sharding_world_size=shards)
    device = torch.device("cuda", torch.cuda.current_device())
    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2, add_bias=False)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=512, add_bias=False)
    config = GPTBaseConfig(vocab_size=1024, hidden_size=256, num_layers=2, position_embedding_type="rope", normalization_function="rmsnorm",
                           max_position_embeddings=256, tie_word_embeddings=False, sequence_mixer_blocks=[attn] * 2, mlp_blocks=[mlp] * 2)
    torch.manual_seed(7)
    model = GPTBaseForCausalLM(config)
    engine = ShardedTrainingEngine(model, compute_dtype=torch.bfloat16, device=device, fused_collectives=fused)
    assert engine.replica_world == replicas and engine.shard_world == shards
    optimizer = FusedAdamW([seg.master for seg in engine.segments()], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    rank = dist.get_rank()
    out = []
    for step in range(3):
        torch.manual_seed(1000 + 10 * step + rank)
        ids = torch.randint(0, 1024, (4, 256), device=device)
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        engine.fold_autograd_grads()
        engine.optimizer_step(optimizer, None, max_norm=1.0)
        value = loss.detach().float()
        dist.all_reduce(value)
        out.append(float(value))
    if engine.peer is not None:
        engine.peer.check()
    ProcessGroupManager.destroy_process_groups()
    return out


def main() -> None:
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    mode = sys.argv[1]
    replicas, shards, fused = {"fsdp4": (1, 4, True), "hsdp-peer": (2, 2, True), "hsdp-nccl": (2, 2, False)}[mode]
    result = losses(replicas, shards, fused)
    if int(os.environ["RANK"]) == 0:
        print("LOSSES " + json.dumps(result), flush=True)


if __name__ == "__main__":
    if len(sys.argv) > 1:
        main()
    else:
        # driver: every topology in its own torchrun job (process groups are built once per process)
        curves = {}
        for index, mode in enumerate(("fsdp4", "hsdp-peer", "hsdp-nccl")):
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr", "127.0.0.1",
                   "--master-port", str(29581 + 2 * index), os.path.abspath(__file__), mode]
            done = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            assert done.returncode == 0, done.stderr[-3000:]
            line = [l for l in done.stdout.splitlines() if l.startswith("LOSSES ")][-1]
            curves[mode] = json.loads(line[len("LOSSES "):])
            print(mode, curves[mode], flush=True)
        for mode in ("hsdp-peer", "hsdp-nccl"):
            for a, b in zip(curves["fsdp4"], curves[mode]):
                assert abs(a - b) <= 2e-3 * max(1.0, abs(a)), (mode, curves)
        print("HSDP_CHECK_OK", flush=True)
