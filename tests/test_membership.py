"""Failure detection of the collective path on the host (no GPU): a rank that leaves between steps, cleanly or
silently, is noticed by the others through the heartbeat store before their next launch."""
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_ranks_that_leave_are_detected_before_the_next_step():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "mp_worker_membership.py"), str(r), "4", str(port)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(4)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    assert all(p.returncode == 0 for p in procs), outs
    for r in (0, 3):
        line = [ln for ln in outs[r].splitlines() if ln.startswith(f"rank {r} events")][0]
        # step 4: rank 2 announced its departure; step 6: rank 1 went silent (time-out); nobody else was lost
        assert "(4, [2], [2])" in line and "(6, [1], [])" in line and "survivors [0, 3]" in line, line
