"""Multi-GPU tests: one process per GPU over NCCL bootstrap + NVLink peer memory."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

HERE = os.path.dirname(os.path.abspath(__file__))


def run_ranks(n, which):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + n), os.path.join(HERE, "mp_worker_gpu.py"), which]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if p.returncode != 0:
        causes = [ln for ln in p.stdout.splitlines() if "WORKER-FAILED" in ln or ln.endswith(" ok")]
        raise AssertionError("\n".join(causes[:4]) or (p.stdout[-1500:] + p.stderr[-1500:]))
    return p.stdout


@pytest.mark.parametrize("which", ["sparse", "dense", "migrate", "aggemm", "dlrm"])
def test_two_ranks(which):
    out = run_ranks(2, which)
    assert f"{which} ok" in out


def test_rank_leaves_between_steps_and_survivor_restores_from_dump(monkeypatch):
    """Host-side failure detection + recovery on real GPUs: no kernel waits for the rank that left."""
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    out = run_ranks(2, "elastic")
    assert "rank 1 left" in out and "elastic ok" in out


def test_all_visible_gpus():
    n = torch.cuda.device_count()
    if n <= 2:
        pytest.skip("covered by the 2-rank test")
    out = run_ranks(n, "all")
    assert "sparse ok" in out and "dense ok" in out and "migrate ok" in out and "aggemm ok" in out and "dlrm ok" in out
