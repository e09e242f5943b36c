"""The service layer across REAL processes: a master process, pserver processes, fault injection by
SIGKILL on the host (the way pico-ps/test/ps_pmem_test.cpp:312-342 kills its pservers), restart in
restore mode."""
import os
import signal
import subprocess
import sys
import time

import numpy as np

from parameter_server_b200 import StatusCode
from parameter_server_b200 import service as S
from test_service import make_table

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def spawn(*args):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.Popen([sys.executable, "-m", "parameter_server_b200.service.launch", *args], stdout=subprocess.PIPE,
                            stderr=subprocess.STDOUT, text=True, env=env, cwd=ROOT)


def test_kill_and_restore_across_processes():
    procs = []
    try:
        master = spawn("master")
        procs.append(master)
        addr = master.stdout.readline().strip()
        assert addr.startswith("127.0.0.1:")
        servers = [spawn("pserver", "--master", addr) for _ in range(3)]
        procs += servers
        ids = [int(s.stdout.readline().split("node_id=")[1].split()[0]) for s in servers]

        class Cl:  # the shape make_table expects
            client = S.Client(addr)

        nodes = {ids[0]: [0, 1], ids[1]: [1, 2], ids[2]: [2, 0]}      # 2x replication
        sid, h = make_table(Cl, nodes)
        push = S.PushHandler(Cl.client, sid, h["push"])
        pull = S.PullHandler(Cl.client, sid, h["pull_ro"])
        keys = np.arange(2000, dtype=np.int64)
        vals = np.ones((2000, 4), np.float32) * (keys[:, None] % 13)
        assert push.async_push(keys, vals).ok()
        # kill one pserver the hard way
        servers[1].send_signal(signal.SIGKILL)
        servers[1].wait(10)
        st, rows = pull.pull(keys, 20000, True)
        assert st.ok() and np.array_equal(rows, vals)
        # restart in restore mode: a new process takes the dead node's place
        fresh = spawn("pserver", "--master", addr, "--restore")
        procs.append(fresh)
        new_id = int(fresh.stdout.readline().split("node_id=")[1].split()[0])
        line = fresh.stdout.readline()
        assert "restore: OK (1 tables)" in line, line
        assert new_id not in ids
        # now lose a second original node: only the restored process still holds shard 1 + 2 copies
        servers[0].send_signal(signal.SIGKILL)
        servers[0].wait(10)
        st, rows = pull.pull(keys, 20000, True)
        assert st.ok() and np.array_equal(rows, vals)
        # orderly shutdown through the EXIT request
        ctl = S.Controller(addr)
        assert ctl.shutdown_node(new_id).ok()
        assert fresh.wait(10) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
