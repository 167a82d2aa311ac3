"""Failures made on the host (CPU ranks over gloo, files on disk): a rank that leaves between steps, a kill switch, a
checkpoint that was never finished. None of these needs or touches a GPU."""

import json
import os
import subprocess
import sys
import time

SCRIPTS = os.path.join(os.path.dirname(__file__), "scripts")


def _env(port: int) -> dict:
    return dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="")


def _torchrun(world: int, port: int, script: str, *args: str) -> list[str]:
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
            "--master-port", str(port), os.path.join(SCRIPTS, script), *args]


def test_a_rank_that_leaves_between_steps_ends_the_others_collective_with_an_error():
    started = time.monotonic()
    done = subprocess.run(_torchrun(2, 29801, "rank_leaves.py"), env=_env(29801), capture_output=True, text=True, timeout=180)
    assert time.monotonic() - started < 150, "the surviving rank hung"
    assert done.returncode != 0
    assert "collective failed after" in done.stdout + done.stderr
    assert "although a rank had left" not in done.stdout + done.stderr


def test_kill_switch_ends_the_job_cleanly_after_the_next_checkpoint(tmp_path):
    save_dir, out = tmp_path / "ckpt", tmp_path / "curve.json"
    save_dir.mkdir()
    (save_dir / "KILLSWITCH").write_text("")
    done = subprocess.run([sys.executable, os.path.join(SCRIPTS, "ckpt_resume.py"), "save", str(save_dir), str(out), "sync"],
                          env=_env(29803), capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert (save_dir / "global_step3").is_dir()
    assert json.loads((save_dir / "latest_checkpointed_iteration.json").read_text())["latest_checkpointed_iteration"] == 3
    assert not out.exists(), "the run went on after the checkpoint although the kill switch was set"


def test_an_unfinished_checkpoint_directory_is_never_resumed_from(tmp_path):
    save_dir = tmp_path / "ckpt"
    a, b = tmp_path / "a.json", tmp_path / "b.json"
    script = os.path.join(SCRIPTS, "ckpt_resume.py")
    subprocess.run([sys.executable, script, "save", str(save_dir), str(a), "sync"], env=_env(29805), check=True, capture_output=True, timeout=600)
    # a later save that died half-way: its directory still carries the temporary name and holds garbage
    broken = save_dir / "global_step5.incomplete"
    (broken / "model").mkdir(parents=True)
    (broken / "model" / "__0_0.distcp").write_bytes(b"\x00" * 100)
    subprocess.run([sys.executable, script, "resume", str(save_dir), str(b), "sync"], env=_env(29807), check=True, capture_output=True, timeout=600)
    first, second = json.loads(a.read_text()), json.loads(b.read_text())
    assert len(second["losses"]) == 2  # resumed from step 3, not from the wreck of step 5
    for x, y in zip(first["losses"], second["losses"]):
        assert abs(x - y) < 2e-5 * max(1.0, abs(x))
