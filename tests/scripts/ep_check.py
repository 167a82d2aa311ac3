"""Expert parallelism against the single-device MoE layer (torchrun, world = expert-parallel size; gloo on CPU, NCCL +
peer memory on GPUs). Every rank owns ``E / ep`` experts and its own tokens; outputs, input gradients, router and
expert gradients must equal those of one device that holds all experts and all tokens. Prints ``EP_CHECK_OK``."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from lm_engine.hf_models.layers.mlp import MoE
from lm_engine.utils import ProcessGroupManager, init_distributed


def build(hidden, inter, experts, top_k, shared=None):
    return MoE(hidden_size=hidden, intermediate_size=inter, shared_intermediate_size=shared, num_experts=experts,
               num_experts_per_tok=top_k, activation_function="swiglu", add_bias=False, dropout=0, init_method="normal",
               initializer_range=0.05, m_width=None, num_layers=2, use_padding_free_transformer=True)


def main():
    world = int(os.environ["WORLD_SIZE"])
    init_distributed(expert_parallel_world_size=world)
    rank = dist.get_rank()
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    from contextlib import nullcontext

    def context():
        if not cuda:
            return nullcontext()
        from lm_engine.enums import Kernel
        from lm_engine.kernels import enable_kernels

        return enable_kernels([Kernel.scattermoe])

    for hidden, inter, experts, top_k, tokens in ((64, 32, 8, 2, 96), (256, 128, 8, 4, 512)) if not cuda else ((512, 256, 8, 2, 1024), (1536, 512, 40, 8, 2048)):
        if experts % world:
            continue
        torch.manual_seed(3)
        local = build(hidden, inter, experts, top_k).to(device=device, dtype=dtype)
        assert local.expert_parallel and local.c_fc.weight.shape[0] == experts // world
        # the single-device layer with the same seed: the expert-parallel layer must hold its slice of these weights
        with _no_ep():
            torch.manual_seed(3)
            full = build(hidden, inter, experts, top_k).to(device=device, dtype=dtype)
        per = experts // world
        assert torch.equal(local.c_fc.weight, full.c_fc.weight[rank * per : (rank + 1) * per])
        assert torch.equal(local.c_proj.weight, full.c_proj.weight[rank * per : (rank + 1) * per])
        assert torch.equal(local.gate.weight, full.gate.weight)

        torch.manual_seed(100)
        x_all = (torch.randn(world * tokens, hidden, device=device) * 0.5).to(dtype)
        dy_all = (torch.randn(world * tokens, hidden, device=device) * 0.1).to(dtype)
        x = x_all[rank * tokens : (rank + 1) * tokens].clone().requires_grad_(True)
        x_ref = x_all.clone().requires_grad_(True)
        with context():
            y = local(x)
            y.backward(dy_all[rank * tokens : (rank + 1) * tokens])
            y_ref = full(x_ref)
            y_ref.backward(dy_all)
        tol = dict(atol=3e-2, rtol=3e-2) if cuda else dict(atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(y.float(), y_ref[rank * tokens : (rank + 1) * tokens].float(), **tol)
        torch.testing.assert_close(x.grad.float(), x_ref.grad[rank * tokens : (rank + 1) * tokens].float(), **tol)
        wtol = dict(atol=0.15, rtol=5e-2) if cuda else dict(atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(local.c_fc.weight.grad.float(), full.c_fc.weight.grad[rank * per : (rank + 1) * per].float(), **wtol)
        torch.testing.assert_close(local.c_proj.weight.grad.float(), full.c_proj.weight.grad[rank * per : (rank + 1) * per].float(), **wtol)
        gate_grad = local.gate.weight.grad.float().clone()
        dist.all_reduce(gate_grad)  # the router is replicated: its gradient is the sum over the ranks' tokens
        torch.testing.assert_close(gate_grad, full.gate.weight.grad.float(), **wtol)
        if cuda:
            from lm_engine import ops

            ops.check_status()
        if rank == 0:
            print(f"ok hidden={hidden} experts={experts} top_k={top_k} tokens/rank={tokens}", flush=True)
    dist.barrier()
    if rank == 0:
        print("EP_CHECK_OK", flush=True)
    dist.destroy_process_group()


class _no_ep:
    """Temporarily report an expert-parallel size of one (to build the single-device layer)."""

    def __enter__(self):
        from lm_engine.utils import parallel

        self.state = parallel._State
        self.saved = self.state.ep_world_size
        self.state.ep_world_size = 1

    def __exit__(self, *exc):
        self.state.ep_world_size = self.saved


if __name__ == "__main__":
    main()
