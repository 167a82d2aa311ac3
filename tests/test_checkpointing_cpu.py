"""Checkpoint layout and resume parity: a run that is interrupted after step 3 and resumed (on the same or on a
different number of ranks) reproduces the losses of steps 4 and 5 of the uninterrupted run."""

import json
import os
import subprocess
import sys

import pytest

SCRIPT = os.path.join(os.path.dirname(__file__), "scripts", "ckpt_resume.py")


def _run(world: int, port: int, *script_args: str, cpu_offload: bool = False):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="",
               TINY_CPU_OFFLOAD="1" if cpu_offload else "0")
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


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_checkpoint_resumes_and_unshards(tmp_path, world):
    """Tensor parallel size 2 (alone, and times two sharding ranks): every rank's block of a split parameter reaches
    the checkpoint, resuming reproduces the uninterrupted losses, and the single-device weights rebuilt from the
    checkpoint equal those of a run without tensor parallelism."""
    import torch

    tp_dir, ref_dir = tmp_path / "tp", tmp_path / "ref"
    a, b, c = tmp_path / "a.json", tmp_path / "b.json", tmp_path / "c.json"
    _run(world, 29711, "save", str(tp_dir), str(a), "sync", "0", "2")
    _run(world, 29713, "resume", str(tp_dir), str(b), "sync", "0", "2")
    first, second = json.loads(a.read_text()), json.loads(b.read_text())
    for x, y in zip(first["losses"], second["losses"]):
        assert abs(x - y) < 2e-5 * max(1.0, abs(x)), (first, second)
    _run(1, 29715, "save", str(ref_dir), str(c), "sync")
    single = json.loads(c.read_text())
    for x, y in zip(first["losses"], single["losses"]):
        assert abs(x - y) < 5e-5 * max(1.0, abs(x)), (first, single)
    _run(1, 29717, "unshard", str(tp_dir), str(tmp_path / "tp.pt"))
    _run(1, 29719, "unshard", str(ref_dir), str(tmp_path / "ref.pt"))
    from_tp, from_ref = torch.load(tmp_path / "tp.pt"), torch.load(tmp_path / "ref.pt")
    assert set(from_tp) == set(from_ref)
    for key, value in from_ref.items():
        assert from_tp[key].shape == value.shape, key
        assert (from_tp[key] - value).abs().max().item() < 1e-4, key


@pytest.mark.parametrize("resume_world,resume_offload", [(2, True), (1, False)])
def test_checkpoint_of_a_cpu_offload_run_resumes_with_and_without_it(tmp_path, resume_world, resume_offload):
    """``cpu_offload`` changes where the master shards and the optimizer state live, not what a checkpoint holds: a run
    saved with it resumes with it, and on another number of ranks without it, with the uninterrupted losses."""
    save_dir = tmp_path / "ckpt"
    a, b = tmp_path / "a.json", tmp_path / "b.json"
    _run(2, 29721, "save", str(save_dir), str(a), "sync", cpu_offload=True)
    _run(resume_world, 29723, "resume", str(save_dir), str(b), "sync", cpu_offload=resume_offload)
    first, second = json.loads(a.read_text()), json.loads(b.read_text())
    assert len(first["losses"]) == len(second["losses"]) == 2
    for x, y in zip(first["losses"], second["losses"]):
        assert abs(x - y) < 2e-5 * max(1.0, abs(x)), (first, second)
