"""Multi-GPU tests of the tensor-parallel path (need >= 2 GPUs; run as child processes, one rank per GPU)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(script: str, mode: str, nproc: int = 2, port: int = 29543, ok: str = "ok"):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, script), mode]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    if proc.returncode != 0:
        # the launcher's summary floods the tail: show the workers' own error lines first
        lines = (proc.stdout + "\n" + proc.stderr).splitlines()
        errs = [ln for ln in lines if "Error" in ln or "WORKER_FAIL" in ln or "assert" in ln.lower()]
        raise AssertionError("\n".join(errs[:40]) + "\n...\n" + proc.stdout[-1500:] + proc.stderr[-1500:])
    assert ok in proc.stdout


def _worlds():
    """Rank counts to test: 2, 4 and 8 as far as the machine has GPUs."""
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    only = [int(w) for w in os.environ.get("DPTB200_TEST_WORLDS", "").split(",") if w]      # e.g. "8": just that size
    return [w for w in (2, 4, 8) if w <= n and (not only or w in only)] or [2]


needs2 = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
@pytest.mark.parametrize("world", _worlds())
def test_fused_gemm_allreduce_peer_loads(world):
    _run("tp_worker.py", "p2p", nproc=world, port=29543, ok="tp_worker ok")


@needs2
@pytest.mark.parametrize("world", _worlds())
def test_fused_gemm_allreduce_auto_multimem(world):
    _run("tp_worker.py", "auto", nproc=world, port=29544, ok="tp_worker ok")


@needs2
@pytest.mark.parametrize("world", _worlds())
@pytest.mark.parametrize("hd", ["64", "128"])
def test_tp_llama_engine_matches_whole_model(hd, world):
    _run("tp_llama_worker.py", hd, nproc=world, port=29545 + (hd == "128"), ok="tp_llama_worker ok")


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_tp_llama_engine_single_rank():
    """The engine as a one-GPU serving path (a group of one rank: no peers, no multicast): same parity check."""
    _run("tp_llama_worker.py", "128", nproc=1, port=29549, ok="tp_llama_worker ok")


@needs2
@pytest.mark.parametrize("world", _worlds())
@pytest.mark.parametrize("cf", ["1.25", "0.5"])
def test_expert_parallel_moe_matches_dense_reference(cf, world):
    _run("ep_worker.py", cf, nproc=world, port=29551 + (cf == "0.5"), ok="ep_worker ok")
