"""Multi-GPU tests of the fused data-parallel path (need >= 2 GPUs; run as child processes, one rank per GPU)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode: str, nproc: int = 2, port: int = 29533):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dp_worker.py"), mode]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "dp_worker ok" in proc.stdout


def _worlds():
    """Rank counts to test: 2, 4 and 8 as far as the machine has GPUs."""
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    only = [int(w) for w in os.environ.get("DPTB200_TEST_WORLDS", "").split(",") if w]      # e.g. "8": just that size
    return [w for w in (2, 4, 8) if w <= n and (not only or w in only)] or [2]


needs2 = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
@pytest.mark.parametrize("world", _worlds())
def test_fused_allreduce_peer_loads(world):
    _run("p2p", nproc=world, port=29533)


@needs2
@pytest.mark.parametrize("world", _worlds())
def test_fused_allreduce_auto_multimem(world):
    _run("auto", nproc=world, port=29534)


@needs2
@pytest.mark.parametrize("world", _worlds())
def test_fused_allreduce_overlapped_with_backward(world):
    _run("overlap", nproc=world, port=29535)


@needs2
def test_fused_allreduce_tolerates_a_late_rank():
    _run("late", nproc=2, port=29536)
