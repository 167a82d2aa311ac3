"""Tensor-parallel models against single-device models on CPU (two gloo ranks): see ``tests/scripts/tp_check.py``."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tensor_parallel_matches_single_device(tmp_path):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29544", os.path.join(ROOT, "tests", "scripts", "tp_check.py")]
    done = subprocess.run(cmd, env=env, cwd=str(tmp_path), capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "TP_CHECK_OK" in done.stdout, (done.stdout[-2000:], done.stderr[-4000:])


def _curve(tmp_path, world: int, port: int, tp: int, sp: int):
    import json

    out = tmp_path / f"curve_{world}_{tp}_{sp}.json"
    script = os.path.join(ROOT, "tests", "scripts", "tiny_pretrain.py")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    if world == 1:
        cmd = [sys.executable, script, str(out), "4", "6", "3"]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), script, str(out), "4", "6", "3", str(tp), str(sp)]
    done = subprocess.run(cmd, env=env, cwd=str(tmp_path), capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-4000:]
    return json.loads(out.read_text())


def test_training_through_the_wrapper_matches_single_process(tmp_path):
    """Pretraining steps with tp=2 + sequence parallelism, and with tp=2 x dp=2, give the single-process loss curve."""
    single = _curve(tmp_path, 1, 0, 1, 0)
    for world, port, tp, sp in ((2, 29551, 2, 1), (4, 29553, 2, 0)):
        other = _curve(tmp_path, world, port, tp, sp)
        for a, b in zip(single, other):
            assert abs(a["loss"] - b["loss"]) < 2e-5 * max(1.0, abs(a["loss"])), (world, tp, sp, single, other)
            assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-4 * max(1.0, abs(a["grad_norm"])), (world, tp, sp, single, other)
