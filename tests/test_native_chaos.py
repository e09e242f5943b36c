"""Rounds of failures against native server processes, in the spirit of the reference's process-level restore test
(pico-ps/test/ps_pmem_test.cpp:367-532: rounds of kill-one / kill-all / lose-the-local-pool followed by a restart in
restore mode, with context updates in between, while a client keeps pulling until it is served and checks values).

Every failure is made on the host: SIGKILL or SIGTERM of a `psb_node pserver` process, or deleting its image files.
Restore sources by round: a live replica (kill one), the host's own images (planned stop of every server), the
table's dump (every server killed and the images gone).
"""
import json
import os
import shutil
import signal
import subprocess
import time

import numpy as np
import pytest

from parameter_server_b200 import _build
from parameter_server_b200 import service as S

NODE = str(_build.node_path())
DIM = 4


def _spawn(*args):
    return subprocess.Popen([NODE, *args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


def _line(p, timeout=30.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        line = p.stdout.readline()
        if line:
            return line.strip()
        if p.poll() is not None:
            break
        time.sleep(0.01)
    raise AssertionError("no output from psb_node")


class Farm:
    def __init__(self, addr, image_dir):
        self.addr, self.image_dir = addr, image_dir
        self.live = {}          # node id -> process
        self.all = []

    def start(self, restore=False, sources=("replica", "image", "dump")):
        args = ["pserver", "--master", self.addr, "--image-dir", self.image_dir]
        if restore:
            args += ["--restore", "--restore-wait", "10", "--restore-pauses-writes"]   # the table is closed to writes while it is copied
        p = _spawn(*args)
        self.all.append(p)
        node = int(_line(p).split("node_id=")[1].split()[0])
        if restore:
            line = _line(p, 60.0)
            assert line.startswith("restore: OK (1 tables) from ") and line.split(" from ")[1] in sources, line
        self.live[node] = p
        return node

    def kill(self, node, sig):
        p = self.live.pop(node)
        p.send_signal(sig)
        out, _ = p.communicate(timeout=30)
        return out

    def close(self):
        for p in self.all:
            if p.poll() is None:
                p.kill()


def _pull_until_served(pull, keys, want, seconds=40.0):
    """The reference's client loop: short timeouts, retry until the cluster serves again, then check the values."""
    t0 = time.time()
    st = None
    while time.time() - t0 < seconds:
        st, rows = pull.pull(keys, 2000, True)
        if st.ok():
            assert np.array_equal(rows, want), np.abs(rows - want).max()
            return
        time.sleep(0.05)
    raise AssertionError(f"not served within {seconds} s: {st}")


def _push_until_applied(push, keys, grads, seconds=40.0):
    t0 = time.time()
    st = None
    while time.time() - t0 < seconds:
        st = push.async_push(keys, grads, 5000)
        if st.ok():
            return
        time.sleep(0.05)
    raise AssertionError(f"push not applied within {seconds} s: {st}")


@pytest.mark.timeout(600)
@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_rounds_of_failures_and_restores(tmp_path):
    master = _spawn("master")
    addr = _line(master)
    farm = Farm(addr, str(tmp_path / "images"))
    try:
        ids = [farm.start() for _ in range(3)]
        client = S.Client(addr)
        # 3 shards x 2 replicas, node i holds shards i and i+1
        place = {ids[i]: [i, (i + 1) % 3] for i in range(3)}
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                        S.storage_config(place, dict(dim=DIM, optimizer="sum", init_range=0.0)))
        assert st.ok(), st
        h = {}
        for key, op, cfg in [("push", "SparseTablePushOperator", {}), ("pull_ro", "SparseTablePullOperator", {"read_only": True}),
                             ("dump", "DumpOperator", {}), ("load", "LoadOperator", {}),
                             ("update_ctx", "ShardUpdateContextOperator", {})]:
            st, h[key] = client.register_handler(key, S.LIB, op, json.dumps(cfg), sid)
            assert st.ok(), st
        uri = str(tmp_path / "dump")
        assert client.set_table_uri(sid, uri).ok()
        push, pull = S.PushHandler(client, sid, h["push"]), S.PullHandler(client, sid, h["pull_ro"])
        keys = np.arange(3000, dtype=np.int64)
        want = np.zeros((3000, DIM), np.float32)
        rng = np.random.default_rng(17)

        def train():
            g = rng.integers(1, 5, size=(3000, 1)).astype(np.float32) * np.ones((1, DIM), np.float32)
            _push_until_applied(push, keys, g)
            want[:] += g

        train()
        _pull_until_served(pull, keys, want)
        plan = ["kill_one", "reshard", "stop_all", "kill_one", "lose_everything", "reshard", "kill_one", "stop_all"]
        for rnd, what in enumerate(plan):
            nodes = sorted(farm.live)
            if what == "kill_one":
                farm.kill(nodes[rnd % len(nodes)], signal.SIGKILL)      # restore source: the live replicas
                farm.start(restore=True, sources=("replica",))
            elif what == "stop_all":
                for n in nodes:                                          # planned stop: every server leaves its images
                    assert "images: OK" in farm.kill(n, signal.SIGTERM)
                farm.start(restore=True, sources=("image",))             # restore source: the host's images (nobody is alive)
                for _ in nodes[1:]:                                      # later ones may find a restored replica first
                    farm.start(restore=True, sources=("image", "replica"))
            elif what == "lose_everything":
                st, n = S.DumpHandler(client, sid, h["dump"]).dump(uri, 2)
                assert st.ok() and n == 3000, st
                for n_ in nodes:
                    farm.kill(n_, signal.SIGKILL)                        # no images are written
                shutil.rmtree(farm.image_dir, ignore_errors=True)        # and whatever was there is gone
                farm.start(restore=True, sources=("dump",))              # restore source: the dump at table_uri
                for _ in nodes[1:]:
                    farm.start(restore=True, sources=("dump", "replica"))
            elif what == "reshard":
                live = sorted(farm.live)
                shift = 1 + rnd % 2
                new_place = {live[i]: [(i + shift) % 3, (i + shift + 1) % 3] for i in range(3)}
                t0 = time.time()
                while True:                                              # the client may first have to learn the new nodes
                    st = S.UpdateContextHandler(client, sid, h["update_ctx"]).update_context(S.nodes_json(new_place))
                    if st.ok() or time.time() - t0 > 30:
                        break
                    client.pull_context(sid)
                    time.sleep(0.2)
                assert st.ok(), st
            _pull_until_served(pull, keys, want)                         # nothing lost, whatever the source was
            train()
            _pull_until_served(pull, keys, want)
            st, info = client.query_storage_info(sid)
            assert st.ok() and sum(i.item_number for i in info) == 2 * 3000, (what, [(i.node_id, i.shard_id, i.item_number) for i in info])
        for n in sorted(farm.live):
            client.close_pserver(n)
        for p in list(farm.live.values()):
            assert p.wait(timeout=20) == 0
        master.send_signal(signal.SIGTERM)
        assert master.wait(timeout=15) == 0
    finally:
        farm.close()
        if master.poll() is None:
            master.kill()


def _read_image(path, stride):
    """Parse a table image; raises when it is torn (short header, short body, trailing bytes)."""
    raw = path.read_bytes()
    assert raw[:8] == b"PSBIMG1\x00", raw[:8]
    ulen = int(np.frombuffer(raw[8:16], "<u8")[0])
    off = 16 + ulen
    width = int(np.frombuffer(raw[off:off + 4], "<u4")[0])
    n = int(np.frombuffer(raw[off + 4:off + 12], "<u8")[0])
    assert width == stride
    rec = np.dtype([("key", "<i8"), ("row", "<f4", (stride,))])
    body = raw[off + 12:]
    assert len(body) == n * rec.itemsize, (len(body), n, rec.itemsize)
    return np.frombuffer(body, rec)


@pytest.mark.timeout(300)
@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_a_killed_server_never_leaves_a_torn_image(tmp_path):
    """Crash consistency of the periodic images (the reference kills a child in the middle of persistent-memory
    transactions and checks invariants afterwards, pico-ps/test/ps_pmem_test.cpp:188-251): a server that refreshes
    its image every few milliseconds is SIGKILLed at random moments under a stream of pushes; whatever is on disk
    afterwards is a complete image whose rows are each from one moment, and a replacement serves it."""
    master = _spawn("master")
    addr = _line(master)
    procs = [master]
    rng = np.random.default_rng(5)
    try:
        client = S.Client(addr)
        img = tmp_path / "images"
        sid = h_push = h_pull = None
        keys = np.arange(2000, dtype=np.int64)
        ones = np.ones((2000, DIM), np.float32)
        pushed = 0
        for rnd in range(4):
            args = ["pserver", "--master", addr, "--image-dir", str(img), "--image-interval-ms", "5"]
            p = _spawn(*(args + (["--restore", "--restore-wait", "10"] if rnd else [])))
            procs.append(p)
            node = int(_line(p).split("node_id=")[1].split()[0])
            if rnd == 0:
                st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                                S.storage_config({node: [0, 1]}, dict(dim=DIM, optimizer="sum", init_range=0.0)))
                assert st.ok(), st
                _, h_push = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
                _, h_pull = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
            else:
                assert _line(p, 60.0) == "restore: OK (1 tables) from image"
                st, rows = S.PullHandler(client, sid, h_pull).pull(keys, 20000, True)
                assert st.ok()
                # the restored state is what the last complete image held: every row from one moment, nothing newer
                # than what was pushed, and not older than the image that was checked on disk
                assert np.all(rows == rows[:, :1]) and rows.max() <= pushed and rows.min() >= floor
                pushed = int(rows.min())            # rows may differ by the pushes that the image caught half-way
                # level the table again so that the next round starts from equal rows
                top = rows[:, :1].max()
                assert S.PushHandler(client, sid, h_push).async_push(keys, (top - rows[:, :1]) * ones, 20000).ok()
                pushed = int(top)
            push = S.PushHandler(client, sid, h_push)
            deadline = time.time() + 0.3 + float(rng.random()) * 0.5
            while time.time() < deadline:
                assert push.async_push(keys, ones, 20000).ok()
                pushed += 1
            p.send_signal(signal.SIGKILL)                       # somewhere between, or inside, two image refreshes
            p.wait(timeout=10)
            path = img / f"node_{node}" / f"storage_{sid}.img"
            assert path.exists()
            image = _read_image(path, DIM)                      # complete: header, count and body agree
            assert len(image) == 2000 and np.all(image["row"] == image["row"][:, :1])
            floor = float(image["row"].min())
            assert floor >= 1 and image["row"].max() <= pushed
        master.send_signal(signal.SIGTERM)
        master.wait(timeout=15)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


def _free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


@pytest.mark.timeout(300)
@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_the_master_is_killed_and_restarted_from_its_state_file(tmp_path):
    """The master keeps ids, contexts and the model registry in a state file. While it is gone the data path goes on
    (clients know the servers' addresses); a new master on the same port reads the file back, the servers register
    again under their node ids and nobody is taken for dead; afterwards everything that needs the master works."""
    port, state = _free_port(), str(tmp_path / "master.state")
    margs = ["master", "--port", str(port), "--state-file", state]
    master = _spawn(*margs)
    procs = [master]
    try:
        addr = _line(master)
        assert addr.endswith(f":{port}")
        servers = [_spawn("pserver", "--master", addr) for _ in range(2)]
        procs += servers
        ids = [int(_line(p).split("node_id=")[1].split()[0]) for p in servers]
        client = S.Client(addr)
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                        S.storage_config({ids[0]: [0], ids[1]: [1]}, dict(dim=DIM, optimizer="sum", init_range=0.0)))
        assert st.ok(), st
        h = {}
        for key, op, cfg in [("push", "SparseTablePushOperator", {}), ("pull_ro", "SparseTablePullOperator", {"read_only": True}),
                             ("update_ctx", "ShardUpdateContextOperator", {})]:
            st, h[key] = client.register_handler(key, S.LIB, op, json.dumps(cfg), sid)
            assert st.ok(), st
        push, pull = S.PushHandler(client, sid, h["push"]), S.PullHandler(client, sid, h["pull_ro"])
        keys = np.arange(1000, dtype=np.int64)
        ones = np.ones((1000, DIM), np.float32)
        assert push.async_push(keys, ones).ok()
        master.send_signal(signal.SIGKILL)
        master.wait(timeout=10)
        # the data path does not need the master
        for _ in range(5):
            assert push.async_push(keys, ones, 5000).ok()
        st, rows = pull.pull(keys, 5000, True)
        assert st.ok() and np.all(rows == 6.0)
        st, _ = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0]}, dict(dim=DIM, optimizer="sum")))
        assert not st.ok()                                          # what needs the master fails cleanly meanwhile
        master2 = _spawn(*margs)
        procs.append(master2)
        assert _line(master2) == addr
        # the servers come back into the registry under their old ids
        t0 = time.time()
        nodes = {}
        while time.time() - t0 < 15:
            st, nodes = client.get_pserver_list()
            if st.ok() and sorted(nodes) == sorted(ids):
                break
            time.sleep(0.2)
        assert sorted(nodes) == sorted(ids), (st, nodes)
        st, rows = pull.pull(keys, 5000, True)
        assert st.ok() and np.all(rows == 6.0)
        # the table's context survived: a reshard (published through the master) works, ids go on where they were
        st = S.UpdateContextHandler(client, sid, h["update_ctx"]).update_context(S.nodes_json({ids[0]: [1], ids[1]: [0]}))
        assert st.ok(), st
        st, rows = pull.pull(keys, 20000, True)
        assert st.ok() and np.all(rows == 6.0)
        st, sid2 = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0]}, dict(dim=DIM, optimizer="sum")))
        assert st.ok() and sid2 > sid
        extra = _spawn("pserver", "--master", addr)
        procs.append(extra)
        new_id = int(_line(extra).split("node_id=")[1].split()[0])
        assert new_id not in ids                                     # node ids are never handed out twice
        for n in ids + [new_id]:
            assert client.close_pserver(n).ok()
        for p in servers + [extra]:
            assert p.wait(timeout=15) == 0
        master2.send_signal(signal.SIGTERM)
        assert master2.wait(timeout=15) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


@pytest.mark.timeout(300)
@pytest.mark.skipif(not os.path.exists(NODE), reason="psb_node is not built")
def test_a_replica_replaced_under_a_stream_of_pushes_is_exact_when_the_restore_pauses_writes():
    """Real processes: one of two replicas is SIGKILLed while a client pushes without a break, a replacement started
    with --restore --restore-pauses-writes copies the table from the survivor, the survivor is killed as well, and the
    replacement alone must hold every push exactly once."""
    import threading
    master = _spawn("master")
    addr = _line(master)
    procs = [master]
    try:
        servers = [_spawn("pserver", "--master", addr) for _ in range(2)]
        procs += servers
        nodes = [int(_line(p).split("node_id=")[1].split()[0]) for p in servers]
        client = S.Client(addr)
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                        S.storage_config({n: [0, 1, 2] for n in nodes}, dict(dim=DIM, optimizer="sum", init_range=0.0)))
        assert st.ok(), st
        _, h_push = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
        _, h_pull = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
        keys = np.arange(30_000, dtype=np.int64)
        ones = np.ones((len(keys), DIM), np.float32)
        stop, applied, bad = threading.Event(), [0], []

        def trainer():
            c = S.Client(addr)
            assert c.initialize_storage(sid).ok()
            push = S.PushHandler(c, sid, h_push)
            while not stop.is_set():
                st_ = push.async_push(keys, ones, 60000)
                if not st_.ok():
                    bad.append(str(st_))
                    return
                applied[0] += 1

        t = threading.Thread(target=trainer)
        t.start()
        try:
            time.sleep(0.3)
            servers[1].send_signal(signal.SIGKILL)
            servers[1].wait(timeout=10)
            before = applied[0]
            fresh = _spawn("pserver", "--master", addr, "--restore", "--restore-wait", "30", "--restore-pauses-writes")
            procs.append(fresh)
            assert "node_id=" in _line(fresh)
            assert _line(fresh, 90.0) == "restore: OK (1 tables) from replica"
            deadline = time.time() + 30
            while time.time() < deadline and applied[0] < before + 3:
                time.sleep(0.05)
            assert applied[0] >= before + 3, (applied, bad)                    # the pushes went on after the pause
        finally:
            stop.set()
            t.join(90)
        assert not bad and not t.is_alive(), bad
        servers[0].send_signal(signal.SIGKILL)                                 # only the replacement is left
        servers[0].wait(timeout=10)
        pull = S.PullHandler(client, sid, h_pull)
        deadline = time.time() + 40
        rows = None
        while time.time() < deadline:
            st, rows = pull.pull(keys, 3000, True)
            if st.ok():
                break
            time.sleep(0.05)
        assert st.ok() and np.all(rows == float(applied[0])), (str(st), float(rows.min()), float(rows.max()), applied[0])
        master.send_signal(signal.SIGTERM)
        master.wait(timeout=15)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
