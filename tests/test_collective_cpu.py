"""The collective API on the host back-end over gloo, 3 ranks, against a single-process oracle."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_sparse_and_dense_tables_over_gloo():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29733", os.path.join(HERE, "mp_worker_cpu.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "cpu collective ok" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]
