"""The native executable (csrc/apps/psb_node.cpp) as master and as parameter servers: a Python client creates a
table on two native server processes, pushes, pulls, loses one server (SIGKILL), starts a replacement in
restore mode and shuts everything down through the admin API. No Python in the serving processes."""
import json
import os
import shutil
import signal
import subprocess
import tempfile
import time

import numpy as np
import pytest

from parameter_server_b200 import _build
from parameter_server_b200 import service as S

NODE = str(_build.node_path())


def _spawn(*args):
    return subprocess.Popen([NODE, *args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


def _first_line(p, timeout=20.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        line = p.stdout.readline()
        if line:
            return line.strip()
        time.sleep(0.01)
    raise AssertionError("no output from psb_node")


@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_native_master_and_servers_serve_a_python_client():
    master = _spawn("master")
    procs = [master]
    try:
        addr = _first_line(master)
        servers = [_spawn("pserver", "--master", addr) for _ in range(2)]
        procs += servers
        ids = [int(_first_line(p).split("node_id=")[1].split()[0]) for p in servers]
        client = S.Client(addr)
        # 2x replication so that the table survives the loss of one process
        cfg = S.storage_config({ids[0]: [0, 1], ids[1]: [0, 1]}, dict(dim=4, optimizer="sum", init_range=0.0))
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", cfg)
        assert st.ok(), st
        st, h_push = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
        assert st.ok()
        st, h_pull = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
        assert st.ok()
        keys = np.arange(1000, dtype=np.int64)
        vals = (keys[:, None] % 7 + 1) * np.ones((1, 4), np.float32)
        assert S.PushHandler(client, sid, h_push).async_push(keys, vals.astype(np.float32)).ok()
        pull = S.PullHandler(client, sid, h_pull)
        st, rows = pull.pull(keys)
        assert st.ok() and np.array_equal(rows, vals)
        # one server process dies the hard way; reads go on from the other replica
        servers[1].send_signal(signal.SIGKILL)
        servers[1].wait(timeout=10)
        for _ in range(8):
            st, rows = pull.pull(keys, 20000, True)
            assert st.ok() and np.array_equal(rows, vals)
        # a replacement restores the lost shards from the live replica
        fresh = _spawn("pserver", "--master", addr, "--restore")
        procs.append(fresh)
        assert "node_id=" in _first_line(fresh)
        assert _first_line(fresh, 30.0) == "restore: OK (1 tables) from replica"
        # admin shutdown: EXIT to every live server, then the master
        st, live = client.get_pserver_list()
        assert st.ok() and len(live) == 2
        for node in live:
            assert client.close_pserver(node).ok()
        for p in (servers[0], fresh):
            assert p.wait(timeout=15) == 0
        master.send_signal(signal.SIGTERM)
        assert master.wait(timeout=15) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_planned_shutdown_leaves_an_image_that_a_replacement_opens(tmp_path):
    master = _spawn("master")
    procs = [master]
    try:
        addr = _first_line(master)
        img = str(tmp_path / "img")
        first = _spawn("pserver", "--master", addr, "--image-dir", img)
        procs.append(first)
        node = int(_first_line(first).split("node_id=")[1].split()[0])
        client = S.Client(addr)
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                        S.storage_config({node: [0, 1]}, dict(dim=4, optimizer="sum", init_range=0.0)))
        assert st.ok(), st
        _, h_push = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
        _, h_pull = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
        keys = np.arange(800, dtype=np.int64)
        vals = ((keys[:, None] % 9 + 1) * np.ones((1, 4))).astype(np.float32)
        assert S.PushHandler(client, sid, h_push).async_push(keys, vals).ok()
        first.send_signal(signal.SIGTERM)                       # planned shutdown: the image is written
        out, _ = first.communicate(timeout=20)
        assert "images: OK (1 tables)" in out and first.returncode == 0
        # the housekeeping verb: the image of a node that is gone is listed, and kept unless asked otherwise
        ls = subprocess.run([NODE, "images", img, "--master", addr, "--remove-unused"], capture_output=True, text=True, timeout=60)
        assert ls.returncode == 0 and "removed=0" in ls.stderr, ls.stderr
        (im,) = json.loads(ls.stdout)
        assert (im["node"], im["storage_id"], im["records"], im["state"]) == (node, sid, 800, "dead_node")
        assert subprocess.run([NODE, "images"], capture_output=True).returncode == 2
        second = _spawn("pserver", "--master", addr, "--image-dir", img, "--restore")
        procs.append(second)
        assert "node_id=" in _first_line(second)
        assert _first_line(second, 30.0) == "restore: OK (1 tables) from image"
        st, rows = S.PullHandler(client, sid, h_pull).pull(keys, 20000, True)
        assert st.ok() and np.array_equal(rows, vals)
        for n in client.get_pserver_list()[1]:
            client.close_pserver(n)
        second.wait(timeout=15)
        master.send_signal(signal.SIGTERM)
        master.wait(timeout=15)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


def _ctl(addr, *args):
    p = subprocess.run([NODE, "ctl", "--master", addr, *args], capture_output=True, text=True, timeout=60)
    return p.returncode, p.stdout.strip(), p.stderr.strip()


@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_controller_from_the_command_line():
    """`psb_node ctl`: create a table on native servers, look at it, resize it, add a node, clean up, shut down."""
    master = _spawn("master")
    procs = [master]
    try:
        addr = _first_line(master)
        servers = [_spawn("pserver", "--master", addr) for _ in range(2)]
        procs += servers
        ids = [int(_first_line(p).split("node_id=")[1].split()[0]) for p in servers]
        rc, out, err = _ctl(addr, "nodes")
        assert rc == 0 and sorted(n["node_id"] for n in json.loads(out)) == sorted(ids), (out, err)
        rc, out, err = _ctl(addr, "create", "emb", "4", "2", json.dumps(dict(dim=4, optimizer="sum", init_range=0.0)))
        assert rc == 0 and out.startswith("storage_id="), (out, err)
        sid = int(out.split("=")[1])
        client = S.Client(addr)
        assert client.initialize_storage(sid).ok()
        push = S.PushHandler(client, sid, client.handler_by_key(sid, "push")[1])
        pull = S.PullHandler(client, sid, client.handler_by_key(sid, "pull_ro")[1])
        keys = np.arange(900, dtype=np.int64)
        vals = ((keys[:, None] % 5 + 1) * np.ones((1, 4))).astype(np.float32)
        assert push.async_push(keys, vals).ok()
        rc, out, err = _ctl(addr, "table", str(sid))
        table = json.loads(out)
        assert rc == 0 and len(table["shards"]) == 8 and sum(s["item_number"] for s in table["shards"]) == 1800   # 4 shards x 2 replicas
        assert _ctl(addr, "shards", str(sid), "6")[0] == 0
        assert _ctl(addr, "replicas", str(sid), "1")[0] == 0
        table = json.loads(_ctl(addr, "table", str(sid))[1])
        assert len(table["shards"]) == 6 and sum(s["item_number"] for s in table["shards"]) == 900
        extra = _spawn("pserver", "--master", addr)
        procs.append(extra)
        new_id = int(_first_line(extra).split("node_id=")[1].split()[0])
        assert _ctl(addr, "expand", str(sid), "2", str(new_id))[0] == 0
        assert _ctl(addr, "balance", str(sid))[0] == 0
        st, rows = pull.pull(keys, 20000, True)
        assert st.ok() and np.array_equal(rows, vals)
        rc, out, err = _ctl(addr, "node", str(new_id))
        assert rc == 0 and json.loads(out)["alive"], (out, err)
        # data verbs: statistics, dump, a second table loaded from the dump, erase by a built-in predicate
        rc, out, err = _ctl(addr, "stats", str(sid))
        stats = json.loads(out)
        assert rc == 0 and stats["count"] == 900 and abs(stats["sum"] - float(vals.sum())) < 1e-3, (out, err)
        dump_dir = tempfile.mkdtemp(prefix="psb_ctl_dump_")
        rc, out, err = _ctl(addr, "dump", str(sid), dump_dir, "2")
        assert rc == 0 and out == "records=900", (out, err)
        rc, out, err = _ctl(addr, "create", "copy", "3", "1", json.dumps(dict(dim=4, optimizer="sum", init_range=0.0)))
        sid2 = int(out.split("=")[1])
        rc, out, err = _ctl(addr, "load", str(sid2), dump_dir)
        assert rc == 0 and out == "records=900", (out, err)
        rc, out, err = _ctl(addr, "erase", str(sid2), json.dumps({"type": "key_mod", "mod": 3, "rem": 0}))
        assert rc == 0 and out == "erased=300", (out, err)
        assert json.loads(_ctl(addr, "stats", str(sid2))[1])["count"] == 600
        assert _ctl(addr, "erase", str(sid2), "{not json")[0] == 1 and _ctl(addr, "dump", str(sid2), dump_dir, "0")[0] == 1
        assert _ctl(addr, "delete", str(sid2))[0] == 0
        shutil.rmtree(dump_dir, ignore_errors=True)
        assert _ctl(addr, "table", "4242")[0] == 1                      # an unknown table is an error, with a message
        assert _ctl(addr, "bogus")[0] == 2
        assert _ctl(addr, "delete", str(sid))[0] == 0
        assert _ctl(addr, "clean")[0] == 0
        for n in ids + [new_id]:
            assert _ctl(addr, "shutdown", str(n))[0] == 0
        for p in servers + [extra]:
            assert p.wait(timeout=15) == 0
        master.send_signal(signal.SIGTERM)
        assert master.wait(timeout=15) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_native_server_exports_prometheus_metrics():
    import urllib.error
    import urllib.request
    master = _spawn("master")
    procs = [master]
    try:
        addr = _first_line(master)
        server = _spawn("pserver", "--master", addr, "--metrics-port", "0")
        procs.append(server)
        node = int(_first_line(server).split("node_id=")[1].split()[0])
        port = int(_first_line(server).split("metrics port=")[1])
        client = S.Client(addr)
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                        S.storage_config({node: [0]}, dict(dim=4, optimizer="sum", init_range=0.0)))
        assert st.ok()
        _, h_push = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
        keys = np.arange(100, dtype=np.int64)
        for _ in range(3):
            assert S.PushHandler(client, sid, h_push).async_push(keys, np.ones((100, 4), np.float32)).ok()
        text = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
        assert f'ps_requests_total{{node_id="{node}",request_type="c2s_async_push",storage_id="{sid}"}} 3' in text
        assert "ps_request_duration_ms_bucket" in text
        with pytest.raises(urllib.error.HTTPError) as ei:
            urllib.request.urlopen(f"http://127.0.0.1:{port}/other", timeout=5)
        assert ei.value.code == 404
        client.close_pserver(node)
        assert server.wait(timeout=15) == 0
        master.send_signal(signal.SIGTERM)
        assert master.wait(timeout=15) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_processes_publish_the_address_they_are_given():
    """--host (or $PSB_HOST): the address a process publishes for its servers. Another loopback address stands in for
    another machine's address here; `localhost` checks that names are resolved."""
    master = _spawn("master", "--host", "127.0.0.2")
    procs = [master]
    try:
        addr = _first_line(master)
        assert addr.startswith("127.0.0.2:")
        server = _spawn("pserver", "--master", addr, "--host", "localhost")
        procs.append(server)
        line = _first_line(server)
        node = int(line.split("node_id=")[1].split()[0])
        assert "c2s=localhost:" in line and "s2s=localhost:" in line
        client = S.Client(addr)
        st, nodes = client.get_pserver_list()
        assert st.ok() and nodes[node].startswith("localhost:")
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                        S.storage_config({node: [0]}, dict(dim=4, optimizer="sum", init_range=0.0)))
        assert st.ok(), st
        _, h_push = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
        _, h_pull = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
        keys = np.arange(64, dtype=np.int64)
        assert S.PushHandler(client, sid, h_push).async_push(keys, np.ones((64, 4), np.float32)).ok()
        st, rows = S.PullHandler(client, sid, h_pull).pull(keys)
        assert st.ok() and np.all(rows == 1.0)
        assert client.close_pserver(node).ok()
        assert server.wait(timeout=15) == 0
        master.send_signal(signal.SIGTERM)
        assert master.wait(timeout=15) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
