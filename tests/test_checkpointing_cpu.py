"""Checkpoint layout and resume parity: a run that is interrupted after step 3 and resumed (on the same or on a
different number of ranks) reproduces the losses of steps 4 and 5 of the uninterrupted run."""

import json
import os
import subprocess
import sys

import pytest

SCRIPT = os.path.join(os.path.dirname(__file__), "scripts", "ckpt_resume.py")


def _run(world: int, port: int, *script_args: str):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="")
    if world == 1:
        cmd = [sys.executable, SCRIPT, *script_args]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
               "127.0.0.1", "--master-port", str(port), SCRIPT, *script_args]
    result = subprocess.run(cmd, env=env, timeout=900, capture_output=True, text=True)
    assert result.returncode == 0, result.stderr[-3000:]


@pytest.mark.parametrize("save_world,resume_world,mode", [(1, 1, "sync"), (2, 1, "sync"), (1, 2, "async")])
def test_resume_reproduces_uninterrupted_losses(tmp_path, save_world, resume_world, mode):
    save_dir = tmp_path / "ckpt"
    a, b = tmp_path / "a.json", tmp_path / "b.json"
    _run(save_world, 29701, "save", str(save_dir), str(a), mode)
    step_dir = save_dir / "global_step3"
    assert (save_dir / "latest_checkpointed_iteration.json").exists()
    assert json.loads((save_dir / "latest_checkpointed_iteration.json").read_text())["latest_checkpointed_iteration"] == 3
    if mode == "async":
        assert (step_dir / "model_optimizer").is_dir()
    else:
        assert (step_dir / "model").is_dir() and (step_dir / "optimizer").is_dir()
    for name in ("lr_scheduler/lr_scheduler-0.pt", "rng_state/rng_state-0.pt", "metadata.json", "training_config.yml"):
        assert (step_dir / name).exists(), name
    _run(resume_world, 29703, "resume", str(save_dir), str(b), mode)
    first, second = json.loads(a.read_text()), json.loads(b.read_text())
    assert len(first["losses"]) == len(second["losses"]) == 2
    for x, y in zip(first["losses"], second["losses"]):
        assert abs(x - y) < 2e-5 * max(1.0, abs(x)), (first, second)
    assert abs(first["lr"] - second["lr"]) < 1e-12
