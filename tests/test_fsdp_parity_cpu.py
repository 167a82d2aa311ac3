"""The tiny gpt_base pretraining config gives the same 20-step loss curve in one process and on two CPU ranks
(gloo) with sharded parameters, gradients and optimizer state."""

import json
import os
import subprocess
import sys

import pytest

SCRIPT = os.path.join(os.path.dirname(__file__), "scripts", "tiny_pretrain.py")


def _run(tmp_path, world: int, port: int, stage: int = 3, sharded_parameters: bool = False, cpu_offload: bool = False):
    out = tmp_path / f"curve_w{world}_s{stage}_{int(sharded_parameters)}{int(cpu_offload)}.json"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="",
               TINY_SHARDED_PARAMETERS="1" if sharded_parameters else "0", TINY_CPU_OFFLOAD="1" if cpu_offload else "0")
    if world == 1:
        cmd = [sys.executable, SCRIPT, str(out), "8", "20", str(stage)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), SCRIPT, str(out), "8", "20", str(stage)]
    subprocess.run(cmd, check=True, env=env, timeout=600, capture_output=True)
    return json.loads(out.read_text())


@pytest.mark.parametrize("stage", [3, 0])
def test_two_rank_loss_curve_matches_single_process(tmp_path, stage):
    single = _run(tmp_path, 1, 29631, stage)
    double = _run(tmp_path, 2, 29633 + stage, stage)
    assert len(single) == len(double) == 20
    for a, b in zip(single, double):
        assert abs(a["loss"] - b["loss"]) < 2e-5 * max(1.0, abs(a["loss"]))
        assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-4 * max(1.0, abs(a["grad_norm"]))
    assert single[-1]["loss"] < single[0]["loss"]


def test_blocks_gathered_and_released_one_by_one_give_the_same_curve(tmp_path):
    """``keep_parameters_gathered: false``: every block's parameters exist in full only during its forward and its
    backward pass, its gradients are reduce-scattered right after its backward pass. Same losses and gradient norms
    as one process, on two and on four ranks."""
    single = _run(tmp_path, 1, 29641, 3)
    for world, port in ((2, 29643), (4, 29645)):
        other = _run(tmp_path, world, port, 3, sharded_parameters=True)
        assert len(single) == len(other) == 20
        for a, b in zip(single, other):
            assert abs(a["loss"] - b["loss"]) < 2e-5 * max(1.0, abs(a["loss"]))
            assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-4 * max(1.0, abs(a["grad_norm"]))


@pytest.mark.parametrize("sharded_parameters", [False, True])
def test_cpu_offload_gives_the_same_curve(tmp_path, sharded_parameters):
    """``distributed_args.cpu_offload``: fp32 master shards and the optimizer's moments live in host memory, the
    gradient shard is staged there and the optimizer runs on the CPU. Same losses and gradient norms as one process
    without it, on two ranks, with the parameters kept gathered and with blocks gathered one by one."""
    single = _run(tmp_path, 1, 29651, 3)
    other = _run(tmp_path, 2, 29653 + int(sharded_parameters), 3, sharded_parameters=sharded_parameters, cpu_offload=True)
    assert len(single) == len(other) == 20
    for a, b in zip(single, other):
        assert abs(a["loss"] - b["loss"]) < 2e-5 * max(1.0, abs(a["loss"]))
        assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-4 * max(1.0, abs(a["grad_norm"]))
