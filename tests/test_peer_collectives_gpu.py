"""Peer-memory collectives: the bounded barrier's timeout on one GPU, and (with two or more GPUs) the multi-rank
checks of ``tests/scripts/peer_check.py`` launched with one process per GPU."""

import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_reports_status():
    """Nobody publishes the second rank's flag, so the wait must end by its own limit with the peer-timeout code and
    leave the context usable."""
    from lm_engine import ops

    C = ops.native()
    device = torch.device("cuda", 0)
    flags = torch.zeros(128, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    table = [flags.data_ptr(), flags[64:].data_ptr()]  # rank 0 is this process; "rank 1" never writes
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    C.peer_barrier(table, 0, 1, 0.25, status)
    end.record()
    torch.cuda.synchronize()
    assert int(status.item()) == 4
    assert 200.0 <= start.elapsed_time(end) <= 2000.0
    # the published flag of this rank is there, the device still works
    assert int(flags[0].item()) == 1 and int(flags[64].item()) == 1
    assert float(torch.ones(8, device=device).sum().item()) == 8.0
    # a barrier whose peers have all arrived passes at once
    status.zero_()
    flags[1] = 2
    C.peer_barrier(table, 0, 2, 0.25, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_collectives_match_nccl():
    world = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, NCCL_DEBUG="WARN")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "scripts", "peer_check.py")]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "PEER_CHECK_OK" in done.stdout, (done.stdout[-3000:], done.stderr[-3000:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_tensor_parallel_gemms_match_nccl():
    world = 2 if torch.cuda.device_count() < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29535", os.path.join(ROOT, "tests", "scripts", "fused_tp_check.py")]
    done = subprocess.run(cmd, env=dict(os.environ, NCCL_DEBUG="WARN"), capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "FUSED_TP_OK" in done.stdout, (done.stdout[-3000:], done.stderr[-3000:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_over_peer_memory_matches_single_device():
    world = 2 if torch.cuda.device_count() < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29537", os.path.join(ROOT, "tests", "scripts", "ep_check.py")]
    done = subprocess.run(cmd, env=dict(os.environ, NCCL_DEBUG="WARN"), capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "EP_CHECK_OK" in done.stdout, (done.stdout[-3000:], done.stderr[-3000:])
