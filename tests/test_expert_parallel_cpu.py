"""Expert parallelism on CPU (two gloo ranks): the layer against the single-device layer, and pretraining steps through
the sharded engine (expert parameters as rank-local units) against a single process."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, CUDA_VISIBLE_DEVICES="")


def _torchrun(world: int, port: int, script: str, *args: str) -> list[str]:
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
            "--master-port", str(port), os.path.join(ROOT, "tests", "scripts", script), *args]


def test_expert_parallel_layer_matches_single_device(tmp_path):
    done = subprocess.run(_torchrun(2, 29581, "ep_check.py"), env=ENV, cwd=str(tmp_path), capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "EP_CHECK_OK" in done.stdout, (done.stdout[-2000:], done.stderr[-4000:])


def test_expert_parallel_training_matches_single_process(tmp_path):
    args = ["8", "4", "3", "1", "0", "1", "1", "none", "1", "sync"]
    single, double = tmp_path / "one.json", tmp_path / "two.json"
    script = os.path.join(ROOT, "tests", "scripts", "tiny_pretrain.py")
    done = subprocess.run([sys.executable, script, str(single), *args, "1"], env=ENV, cwd=str(tmp_path), capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-4000:]
    done = subprocess.run(_torchrun(2, 29585, "tiny_pretrain.py", str(double), *args, "2"), env=ENV, cwd=str(tmp_path), capture_output=True,
                          text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-4000:]
    for a, b in zip(json.loads(single.read_text()), json.loads(double.read_text())):
        assert abs(a["loss"] - b["loss"]) < 2e-5 * max(1.0, abs(a["loss"]))
        assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-4 * max(1.0, abs(a["grad_norm"]))


def test_expert_parallel_checkpoint_resume(tmp_path):
    """Save after 3 steps with the experts spread over two ranks, resume, and get the losses of the uninterrupted run."""
    save_dir, a, b = tmp_path / "ckpt", tmp_path / "a.json", tmp_path / "b.json"
    for phase, port, out in (("save", 29587, a), ("resume", 29589, b)):
        done = subprocess.run(_torchrun(2, port, "ckpt_resume.py", phase, str(save_dir), str(out), "sync", "2"), env=ENV, cwd=str(tmp_path),
                              capture_output=True, text=True, timeout=900)
        assert done.returncode == 0, done.stderr[-4000:]
    first, second = json.loads(a.read_text()), json.loads(b.read_text())
    assert len(first["losses"]) == len(second["losses"]) == 2
    for x, y in zip(first["losses"], second["losses"]):
        assert abs(x - y) < 2e-5 * max(1.0, abs(x)), (first, second)
