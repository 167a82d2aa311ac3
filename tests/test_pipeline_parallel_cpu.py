"""Pipeline parallelism: every schedule is a valid order (simulated), and training through the pipeline reproduces the
single-process loss curve on CPU."""

import json
import os
import subprocess
import sys

import pytest

from lm_engine.parallel.pipeline import BACKWARD, FORWARD, build_actions

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("schedule,world,stages,micro", [
    ("GPipe", 1, 1, 3), ("GPipe", 2, 2, 4), ("GPipe", 2, 4, 4), ("GPipe", 4, 8, 8),
    ("1F1B", 2, 2, 1), ("1F1B", 2, 2, 4), ("1F1B", 4, 4, 8), ("1F1B", 4, 4, 2),
    ("Interleaved1F1B", 2, 4, 4), ("Interleaved1F1B", 4, 8, 8), ("Interleaved1F1B", 4, 16, 4), ("Interleaved1F1B", 2, 2, 4),
])
def test_schedules_are_complete_and_free_of_deadlock(schedule, world, stages, micro):
    """Run all ranks' action lists against each other: an action may start when the action it depends on has finished
    (forward of the previous stage, backward of the next stage, own forward before own backward)."""
    lists = [build_actions(schedule, r, world, stages, micro) for r in range(world)]
    for r, actions in enumerate(lists):
        assert len(actions) == len(set(actions)) == 2 * micro * stages // world
        assert all(stage % world == r for _, stage, _ in actions)
    done = set()
    cursor = [0] * world
    progressed = True
    while progressed:
        progressed = False
        for r in range(world):
            while cursor[r] < len(lists[r]):
                kind, stage, m = lists[r][cursor[r]]
                if kind == FORWARD:
                    ready = stage == 0 or (FORWARD, stage - 1, m) in done
                else:
                    ready = (FORWARD, stage, m) in done and (stage == stages - 1 or (BACKWARD, stage + 1, m) in done)
                if not ready:
                    break
                done.add((kind, stage, m))
                cursor[r] += 1
                progressed = True
    assert all(cursor[r] == len(lists[r]) for r in range(world)), f"stuck at {[l[c] if c < len(l) else None for l, c in zip(lists, cursor)]}"
    if schedule != "GPipe" and micro >= world:
        # the point of 1F1B: the first stage never holds more than `depth` forward results waiting for a backward
        depth = world if stages == world else 2 * (world - 1) + (stages // world - 1) * world + 1
        live = peak = 0
        for kind, _, _ in lists[0]:
            live += 1 if kind == FORWARD else -1
            peak = max(peak, live)
        assert peak <= depth


def _curve(tmp_path, world, port, tp, sp, pp, stages, schedule, ga):
    out = tmp_path / f"curve_{world}_{tp}_{pp}_{schedule}.json"
    script = os.path.join(ROOT, "tests", "scripts", "tiny_pretrain.py")
    args = [str(out), "8", "4", "3", str(tp), str(sp), str(pp), str(stages), schedule, str(ga), "sync"]
    if world == 1:
        cmd = [sys.executable, script] + args
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), script] + args
    done = subprocess.run(cmd, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""), cwd=str(tmp_path), capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-4000:]
    return json.loads(out.read_text())


def test_pipeline_training_matches_single_process(tmp_path):
    single = _curve(tmp_path, 1, 0, 1, 0, 1, 1, "none", 4)
    for world, port, tp, sp, pp, schedule in ((2, 29571, 1, 0, 2, "1F1B"), (4, 29573, 2, 1, 2, "GPipe")):
        other = _curve(tmp_path, world, port, tp, sp, pp, pp, schedule, 4)
        for a, b in zip(single, other):
            assert abs(a["loss"] - b["loss"]) < 2e-5 * max(1.0, abs(a["loss"])), (schedule, single, other)
            assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-4 * max(1.0, abs(a["grad_norm"])), (schedule, single, other)
