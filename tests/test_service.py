"""Service layer end to end on CPU: master, servers, clients, handlers, controller, HA, reshard.

Modelled on pico-ps/test/ps_service_test.cpp:77-498, ps_ha_loader_puller_test.cpp:34-238 and
ps_predictor_native_ps_test.cpp:74-191: every "node" is a real server with its own sockets on
localhost; failures are injected on the host (a server is stopped, a memory limit is lowered)."""
import json
import threading
import time

import numpy as np
import pytest

from parameter_server_b200 import C, StatusCode
from parameter_server_b200 import service as S

DIM = 4


def op_cfg(**kw):
    d = dict(dim=DIM, optimizer="sum", init_range=0.0)
    d.update(kw)
    return d


class Cluster:
    def __init__(self, n):
        self.master = S.Master()
        self.servers = [S.Server(self.master.address()) for _ in range(n)]
        self.client = S.Client(self.master.address())

    def ids(self):
        return [s.node_id() for s in self.servers]

    def close(self):
        for s in self.servers:
            s.stop()
        self.master.stop()


@pytest.fixture
def cluster3():
    c = Cluster(3)
    yield c
    c.close()


def make_table(cl, nodes, cfg=None, compress=""):
    st, sid = cl.client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config(nodes, cfg or op_cfg()))
    assert st.ok(), st
    hids = {}
    for spec_key, op, c in [("pull", "SparseTablePullOperator", {}), ("pull_ro", "SparseTablePullOperator", {"read_only": True}),
                            ("push", "SparseTablePushOperator", {}), ("for_each", "ForEachOperator", {}),
                            ("erase_if", "EraseIfOperator", {}), ("dump", "DumpOperator", {"compress_algorithm": compress}),
                            ("load", "LoadOperator", {"compress_algorithm": compress, "block_size": 100}),
                            ("update_ctx", "ShardUpdateContextOperator", {}), ("sync", "KVSyncOperator", {"compress_algorithm": compress})]:
        st, hid = cl.client.register_handler(spec_key, S.LIB, op, json.dumps(c), sid)
        assert st.ok(), st
        hids[spec_key] = hid
    return sid, hids


def uneven(ids):
    """node i owns i+2 shards (the reference's test placement)."""
    out, s = {}, 0
    for i, n in enumerate(ids):
        out[n] = list(range(s, s + i + 2))
        s += i + 2
    return out


def test_a_node_that_registers_again_is_not_wiped_by_the_close_of_its_old_session():
    """A server whose connection to the master broke registers again over a new one. The master may notice the close
    of the old connection only afterwards: the entry belongs to the new session by then and stays."""
    m = S.Master()
    try:
        old, new, reader = (S.MasterClient(m.address()) for _ in range(3))
        st, nid = old.register_node("svc", "127.0.0.1:1")
        assert st.ok() and reader.get_nodes("svc")[1] == {nid: "127.0.0.1:1"}
        st, same = new.register_node("svc", "127.0.0.1:2", nid)          # the same node, over another connection
        assert st.ok() and same == nid
        old.close()                                                        # noticed after the new registration
        for _ in range(20):
            time.sleep(0.02)
            assert reader.get_nodes("svc")[1] == {nid: "127.0.0.1:2"}
        new.close()                                                        # the session that owns the entry: now it goes
        deadline = time.time() + 5
        while time.time() < deadline and reader.get_nodes("svc")[1]:
            time.sleep(0.02)
        assert reader.get_nodes("svc")[1] == {}
    finally:
        m.stop()


def test_a_client_that_lost_the_lock_with_its_connection_cannot_undo_the_holders_work():
    """The global lock belongs to a connection. A client whose connection broke in the middle of its critical section
    comes back over a new one without the lock: its late release leaves the new holder's lock alone, and its write
    to a table context is refused while somebody else holds the lock."""
    m = S.Master()
    try:
        a, b, c = (S.MasterClient(m.address()) for _ in range(3))
        assert a.set_context("storage/7", "v0").ok()                      # nobody holds the lock: tools may edit
        assert a.acquire_lock("PSERVER_LOCK").ok()
        a.close()                                                          # the fault: the lock goes with the connection
        assert b.acquire_lock("PSERVER_LOCK").ok()                        # somebody else is in the critical section now
        assert b.set_context("storage/7", "by the holder").ok()
        st = a.set_context("storage/7", "by the one who lost it")         # over a new connection, unaware
        assert not st.ok() and "lock" in str(st)
        assert not a.delete_context("storage/7").ok()
        assert a.set_context("model/x", "not a table context").ok()        # other keys are not under the lock
        assert a.release_lock("PSERVER_LOCK").ok()                        # a no-op: it is not a's lock
        got = []
        t = threading.Thread(target=lambda: got.append(c.acquire_lock("PSERVER_LOCK").ok()))
        t.start()
        time.sleep(0.3)
        assert t.is_alive() and not got                                    # b still holds it: c waits
        assert b.get_context("storage/7")[1] == "by the holder"
        assert b.release_lock("PSERVER_LOCK").ok()
        t.join(10)
        assert got == [True]
        assert c.release_lock("PSERVER_LOCK").ok()
    finally:
        m.stop()


def test_a_participant_that_went_away_no_longer_stands_at_its_barrier():
    m = S.Master()
    try:
        a, b, c = (S.MasterClient(m.address()) for _ in range(3))
        res = {}
        ta = threading.Thread(target=lambda: res.__setitem__("a", a.barrier("sync", 2)))
        ta.start()
        time.sleep(0.2)
        a.close()                                                          # a waits at the barrier and is lost
        ta.join(10)
        assert not ta.is_alive() and not res["a"].ok()
        tb = threading.Thread(target=lambda: res.__setitem__("b", b.barrier("sync", 2)))
        tb.start()
        time.sleep(0.4)
        assert tb.is_alive()                                               # b alone does not complete it with a's ghost
        assert c.barrier("sync", 2).ok()
        tb.join(10)
        assert res["b"].ok()
    finally:
        m.stop()


def test_master_basics():
    m = S.Master()
    a, b = S.MasterClient(m.address()), S.MasterClient(m.address())
    assert a.generate_id("x")[1] == 0 and b.generate_id("x")[1] == 1 and a.generate_id("y")[1] == 0
    assert a.set_context("k", "v1").ok()
    assert not a.set_context("k", "v2", True).ok()
    assert b.get_context("k")[1] == "v1"
    assert b.get_context("missing")[0].code() == StatusCode.INVALID_ID
    # the lock is exclusive and handed over in order
    order = []
    assert a.acquire_lock("L").ok()
    t = threading.Thread(target=lambda: (b.acquire_lock("L"), order.append("b"), b.release_lock("L")))
    t.start()
    time.sleep(0.1)
    order.append("a")
    a.release_lock("L")
    t.join(5)
    assert order == ["a", "b"]
    # registry membership is liveness: closing the session unregisters the node
    st, nid = a.register_node("svc", "127.0.0.1:1")
    assert st.ok() and b.get_nodes("svc")[1] == {nid: "127.0.0.1:1"}
    a.close()
    for _ in range(50):
        if b.get_nodes("svc")[1] == {}:
            break
        time.sleep(0.05)
    assert b.get_nodes("svc")[1] == {}
    # barrier of 3
    cs = [S.MasterClient(m.address()) for _ in range(3)]
    done = []
    ts = [threading.Thread(target=lambda c=c: done.append(c.barrier("bar", 3).ok())) for c in cs]
    [t.start() for t in ts]
    [t.join(5) for t in ts]
    assert done == [True] * 3
    assert b.tree_node_set("p/q", "1").ok() and b.tree_node_get("p/q")[1] == "1"
    m.stop()


@pytest.mark.parametrize("n_servers", [1, 3, 5, 8])     # the reference's matrix: {1, 3, 5, 8} processes x compression
@pytest.mark.parametrize("compress", ["", "zstd", "lz4"])
def test_sparse_end_to_end(tmp_path, n_servers, compress):
    cl = Cluster(n_servers)
    try:
        sid, h = make_table(cl, uneven(cl.ids()), compress=compress)
        pull, push = S.PullHandler(cl.client, sid, h["pull"]), S.PushHandler(cl.client, sid, h["push"])
        keys = np.arange(2000, dtype=np.int64)
        g = np.tile(np.arange(1, DIM + 1, dtype=np.float32), (2000, 1)) * (keys[:, None] % 7 + 1)
        assert push.async_push(keys, g).ok()
        assert push.async_push(keys[:500], g[:500]).ok()            # extra pushes on a subset
        both = np.concatenate([keys, keys[:100]])                     # duplicates are pre-aggregated client-side
        assert push.async_push(both, np.concatenate([g, g[:100]])).ok()
        exp = g * 2
        exp[:500] += g[:500]
        exp[:100] += g[:100]
        st, rows = pull.pull(keys)
        assert st.ok() and np.array_equal(rows, exp)
        st, info = cl.client.query_storage_info(sid)
        assert st.ok() and sum(i.item_number for i in info) == 2000
        assert len(info) == sum(len(v) for v in uneven(cl.ids()).values())
        # dump with 2 files per node, delete, recreate with a different sharding, load (rehash)
        uri = str(tmp_path / "dump") + "?format=binary"
        st, n = S.DumpHandler(cl.client, sid, h["dump"]).dump(uri, 2)
        assert st.ok() and n == 2000
        assert cl.client.delete_storage(sid).ok()
        other = {n_: [i] for i, n_ in enumerate(cl.ids())}
        sid2, h2 = make_table(cl, other, compress=compress)
        st, n = S.LoadHandler(cl.client, sid2, h2["load"]).load(uri)
        assert st.ok() and n == 2000, st
        pull2 = S.PullHandler(cl.client, sid2, h2["pull_ro"])
        st, rows = pull2.pull(keys[::-1].copy())
        assert st.ok() and np.array_equal(rows, exp[::-1])
        # for_each statistics, erase_if(odd keys), verify
        st, r = S.ForEachHandler(cl.client, sid2, h2["for_each"]).for_each("{}")
        assert st.ok() and r["count"] == 2000 and abs(r["sum"] - float(exp.sum())) < 1e-3 * abs(exp.sum())
        st, erased = S.EraseIfHandler(cl.client, sid2, h2["erase_if"]).erase_if(json.dumps({"type": "key_mod", "mod": 2, "rem": 1}))
        assert st.ok() and erased == 1000
        st, rows = pull2.pull(keys)
        assert np.array_equal(rows[::2], exp[::2]) and np.all(rows[1::2] == 0)   # read-only pull of a missing key = init value
        assert sum(s.storage_size(sid2) for s in cl.servers) == 1000
        # clear
        assert cl.client.clear_storage(sid2).ok()
        assert sum(s.storage_size(sid2) for s in cl.servers) == 0
    finally:
        cl.close()


def test_text_dump_round_trip_is_bitwise(tmp_path, cluster3):
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()), cfg=op_cfg(optimizer="adagrad", lr=0.05, init_accumulator=0.1, init_range=0.01))
    pull, push = S.PullHandler(cl.client, sid, h["pull"]), S.PushHandler(cl.client, sid, h["push"])
    rng = np.random.default_rng(0)
    keys = rng.integers(0, 1 << 40, size=3000)
    pull.pull(keys)
    assert push.async_push(keys, rng.standard_normal((3000, DIM)).astype(np.float32) * 1e-3).ok()
    st, before = pull.pull(keys)
    for fmt in ("archiveline", "binary"):
        uri = str(tmp_path / fmt) + "?format=" + fmt
        assert S.DumpHandler(cl.client, sid, h["dump"]).dump(uri, 3)[0].ok()
        sid2, h2 = make_table(cl, {cl.ids()[0]: [0, 1]}, cfg=op_cfg(optimizer="adagrad", lr=0.05, init_accumulator=0.1, init_range=0.01))
        st, n = S.LoadHandler(cl.client, sid2, h2["load"]).load(uri)
        assert st.ok() and n == len(set(keys.tolist()))
        st, after = S.PullHandler(cl.client, sid2, h2["pull_ro"]).pull(keys)
        assert st.ok() and after.tobytes() == before.tobytes()
        # restore (no rehash) needs the dump's sharding: same placement as the source
        sid3, h3 = make_table(cl, uneven(cl.ids()), cfg=op_cfg(optimizer="adagrad", lr=0.05, init_accumulator=0.1, init_range=0.01))
        st, n = S.LoadHandler(cl.client, sid3, h3["load"]).restore(uri)
        assert st.ok() and n == len(set(keys.tolist()))
        st, again = S.PullHandler(cl.client, sid3, h3["pull_ro"]).pull(keys)
        assert again.tobytes() == before.tobytes()


def test_sync_push_store_and_dense(cluster3):
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()), cfg=op_cfg(sync=True))
    pull, push = S.PullHandler(cl.client, sid, h["pull"]), S.PushHandler(cl.client, sid, h["push"])
    keys = np.arange(300, dtype=np.int64)
    g = np.ones((300, DIM), np.float32)
    assert push.sync_push(keys, g).ok() and push.sync_push(keys, 2 * g).ok()
    assert np.all(pull.pull(keys)[1] == 0)         # buffered, not applied
    assert push.store().ok()
    assert np.all(pull.pull(keys)[1] == 3)
    # dense table: tensors cut into slices of `dim`, slice -> shard by hash % N
    st, dsid = cl.client.create_storage(S.LIB, "DenseTableStorageOperator", S.storage_config(uneven(cl.ids()), op_cfg(dim=5)))
    assert st.ok()
    _, hp = cl.client.register_handler("pull", S.LIB, "DenseTablePullOperator", "{}", dsid)
    _, hq = cl.client.register_handler("push", S.LIB, "DenseTablePushOperator", "{}", dsid)
    dpull, dpush = S.PullHandler(cl.client, dsid, hp), S.PushHandler(cl.client, dsid, hq)
    for tid in (1, 2, 3):
        n = 7 * tid + 3
        v = np.arange(n, dtype=np.float32) + tid
        assert dpush.push_dense(tid, v).ok() and dpush.push_dense(tid, v).ok()
        st, got = dpull.pull_dense(tid, n)
        assert st.ok() and np.array_equal(got, 2 * v)
    st, info = cl.client.query_storage_info(dsid)
    assert len({i.node_id for i in info if i.item_number}) > 1     # slices are spread over the servers


def test_context_version_gate_and_auto_refresh(cluster3):
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()))
    other = S.Client(cl.master.address())
    assert other.initialize_storage(sid).ok()
    pull = S.PullHandler(other, sid, h["pull"])
    assert pull.pull(np.arange(10))[0].ok()
    # the first client changes the context (table uri): `other` is now behind
    assert cl.client.set_table_uri(sid, "/tmp/nowhere").ok()
    st, _ = pull.pull(np.arange(10), 5000, False)
    assert st.code() == StatusCode.SERVER_TOO_NEW_CTX
    st, _ = pull.pull(np.arange(10), 5000, True)          # auto retry refreshes the context
    assert st.ok() and pull.metrics()["retries"] >= 1
    # attaching by key
    st, hid = other.handler_by_key(sid, "push")
    assert st.ok() and hid == h["push"]


def test_update_context_reshard_keeps_data_and_blocks_writes(cluster3):
    cl = cluster3
    ids = cl.ids()
    sid, h = make_table(cl, {ids[0]: [0, 1], ids[1]: [2]})
    pull_ro = S.PullHandler(cl.client, sid, h["pull_ro"])
    push = S.PushHandler(cl.client, sid, h["push"])
    keys = np.arange(5000, dtype=np.int64)
    vals = (keys[:, None] + np.arange(DIM)[None]).astype(np.float32)
    assert push.async_push(keys, vals).ok()
    # a reader keeps pulling while the table is resharded 3 -> 6 shards over all three nodes
    stop, errors = threading.Event(), []
    reader = S.Client(cl.master.address())
    reader.initialize_storage(sid)
    rp = S.PullHandler(reader, sid, h["pull_ro"])

    def read_loop():
        while not stop.is_set():
            st, rows = rp.pull(keys[:200], 10000, True)
            if not st.ok() or not np.array_equal(rows, vals[:200]):
                errors.append(str(st))

    t = threading.Thread(target=read_loop)
    t.start()
    new = {ids[0]: [0, 3], ids[1]: [1, 4], ids[2]: [2, 5]}
    st = S.UpdateContextHandler(cl.client, sid, h["update_ctx"]).update_context(S.nodes_json(new))
    stop.set()
    t.join(10)
    assert st.ok(), st
    assert errors == []
    st, rows = pull_ro.pull(keys)
    assert st.ok() and np.array_equal(rows, vals)
    st, info = cl.client.query_storage_info(sid)
    assert sorted(i.shard_id for i in info) == list(range(6)) and sum(i.item_number for i in info) == 5000
    assert {i.node_id for i in info} == set(ids)
    # writes work again after the transaction
    assert push.async_push(keys[:10], vals[:10]).ok()
    assert np.array_equal(pull_ro.pull(keys[:10])[1], 2 * vals[:10])
    # while a table is in RESHARD, writes are refused with OUT_OF_MEMORY and read-only pulls go on
    td = S.TableDescriptor()
    td.from_json_str(cl.client.get_current_ctx(sid)[1])
    assert td.create_update_info(S.nodes_json(new)).ok()
    mc = S.MasterClient(cl.master.address())
    assert mc.set_context(f"storage/{sid}", td.to_json_str()).ok()
    assert cl.client.pull_context(sid).ok()
    assert cl.client.notify_ctx_update(sid).ok()      # tell the servers
    w = S.Client(cl.master.address())
    w.initialize_storage(sid)
    wp = S.PushHandler(w, sid, h["push"])
    st = wp.async_push(keys[:5], vals[:5], 1500)
    assert st.code() in (StatusCode.OUT_OF_MEMORY, StatusCode.TIMEOUT, StatusCode.SERVER_TOO_OLD_CTX), st
    assert S.PullHandler(w, sid, h["pull_ro"]).pull(keys[:5], 5000)[0].ok()
    # the abort path cleans up
    assert S.UpdateContextHandler(w, sid, h["update_ctx"]).purge().ok()
    assert wp.async_push(keys[:5], vals[:5], 5000).ok()


def test_ha_dead_node_detection_and_restore(tmp_path):
    cl = Cluster(3)
    try:
        ids = cl.ids()
        # 2x replication: every shard on two nodes
        nodes = {ids[0]: [0, 1], ids[1]: [1, 2], ids[2]: [2, 0]}
        sid, h = make_table(cl, nodes)
        push = S.PushHandler(cl.client, sid, h["push"])
        pull = S.PullHandler(cl.client, sid, h["pull_ro"])
        keys = np.arange(3000, dtype=np.int64)
        vals = np.ones((3000, DIM), np.float32) * (keys[:, None] % 11)
        assert push.async_push(keys, vals).ok()              # pushes update every replica
        assert sum(s.storage_size(sid) for s in cl.servers) == 6000
        # node 1 dies (host-side fault: the process' server object is stopped)
        cl.servers[1].stop()
        # a pull picks one replica per shard at random: it meets the dead node after a few pulls at most, then
        # timeout -> dead-node detection -> retry on the other replica, all inside the handler
        td = S.TableDescriptor()
        for _ in range(64):
            st, rows = pull.pull(keys, 20000, True)
            assert st.ok() and np.array_equal(rows, vals)
            td.from_json_str(S.MasterClient(cl.master.address()).get_context(f"storage/{sid}")[1])
            if td.node_status()[ids[1]] == 1:
                break
        assert td.node_status()[ids[1]] == 1                 # DEAD, published on the master
        # a fresh server takes over the dead node's shards from the live replicas
        fresh = S.Server(cl.master.address())
        cl.servers.append(fresh)
        st, n = fresh.restore_storages()
        assert st.ok() and n == 1, st
        assert fresh.node_id() not in ids                    # node ids are never reused
        assert fresh.storage_size(sid) == cl.servers[1].storage_size(sid) or fresh.storage_size(sid) > 0
        td.from_json_str(S.MasterClient(cl.master.address()).get_context(f"storage/{sid}")[1])
        assert td.node_status()[fresh.node_id()] == 0        # RUNNING
        # lose another original node: the restored one must now serve its shards
        cl.servers[0].stop()
        st, rows = pull.pull(keys, 20000, True)
        assert st.ok() and np.array_equal(rows, vals)
    finally:
        cl.close()


def test_scans_of_a_live_table_see_every_old_key_exactly_once(tmp_path):
    """Dumps and a replica restore run while another client keeps inserting new keys, which makes the shard's index
    rebuild itself several times. A dump reads each shard as one snapshot (writers of the shard wait), the resumable
    restore iteration starts over when the index moved under its cursor: no key that was there before is lost or
    written twice."""
    cl = Cluster(2)
    try:
        ids = cl.ids()
        sid, h = make_table(cl, {ids[0]: [0], ids[1]: [0]})                   # one shard, two replicas
        push = S.PushHandler(cl.client, sid, h["push"])
        old = np.arange(60_000, dtype=np.int64)
        assert push.async_push(old, np.ones((len(old), DIM), np.float32)).ok()
        stop, pushed, bad = threading.Event(), [len(old)], []

        def feeder():
            c = S.Client(cl.master.address())
            assert c.initialize_storage(sid).ok()
            q = S.PushHandler(c, sid, h["push"])
            while not stop.is_set() and pushed[0] < 1_500_000:
                k = np.arange(pushed[0], pushed[0] + 10_000, dtype=np.int64)
                st = q.async_push(k, 2 * np.ones((len(k), DIM), np.float32), 20000)
                if not st.ok():
                    bad.append(str(st))
                    return
                pushed[0] += len(k)

        t = threading.Thread(target=feeder)
        t.start()
        try:
            for i in range(4):
                before = pushed[0]
                uri = str(tmp_path / f"dump{i}") + "?format=binary"
                st, n = S.DumpHandler(cl.client, sid, h["dump"]).dump(uri, 1)
                assert st.ok(), st
                assert n >= before                                            # one replica dumps the shard
                sid2, h2 = make_table(cl, {ids[0]: [0, 1]})
                st, loaded = S.LoadHandler(cl.client, sid2, h2["load"]).load(uri)
                assert st.ok(), st
                st, rows = S.PullHandler(cl.client, sid2, h2["pull_ro"]).pull(old)
                assert st.ok() and np.all(rows == 1.0)                        # nothing old is missing
                st, info = cl.client.query_storage_info(sid2)
                uniq = sum(x.item_number for x in info)
                assert uniq == n == loaded                                    # and the snapshot holds no key twice
                assert cl.client.delete_storage(sid2).ok()
            # replica restore in small batches while the inserts go on
            cl.servers[1].stop()
            pull = S.PullHandler(cl.client, sid, h["pull_ro"])
            td = S.TableDescriptor()
            for _ in range(64):
                assert pull.pull(old[:100], 20000, True)[0].ok()
                td.from_json_str(S.MasterClient(cl.master.address()).get_context(f"storage/{sid}")[1])
                if td.node_status()[ids[1]] == 1:
                    break
            assert td.node_status()[ids[1]] == 1
            cfg = S.ServerConfig()
            cfg.restore_batch_size = 4096
            fresh = S.Server(cl.master.address(), cfg)
            cl.servers.append(fresh)
            grown = pushed[0]
            st, n = fresh.restore_storages()
            assert st.ok() and n == 1, st
        finally:
            stop.set()
            t.join(60)
        assert not bad and not t.is_alive(), bad
        assert pushed[0] > grown or pushed[0] >= 1_500_000                    # the inserts did go on during the restore
        cl.servers[0].stop()                                                  # only the restored replica is left
        st, rows = pull.pull(old, 20000, True)
        assert st.ok() and np.all(rows == 1.0)
    finally:
        cl.close()


def test_writing_for_each_updates_every_replica_in_place(cluster3):
    """The writing scan (the reference's SparseTableForEachWriteOperator): every holder of a shard applies it, so
    replicas stay alike; the result counts each shard once; bad carried items are refused before anything changes."""
    cl = cluster3
    ids = cl.ids()
    cfg = op_cfg(optimizer="adagrad", lr=0.1, init_accumulator=0.5)
    sid, h = make_table(cl, {ids[0]: [0, 1], ids[1]: [1, 2], ids[2]: [2, 0]}, cfg=cfg)
    st, hw = cl.client.register_handler("for_each_write", S.LIB, "ForEachWriteOperator", "{}", sid)
    assert st.ok(), st
    push, pull = S.PushHandler(cl.client, sid, h["push"]), S.PullHandler(cl.client, sid, h["pull_ro"])
    keys = np.arange(1, 2001, dtype=np.int64)
    assert push.async_push(keys, np.ones((2000, DIM), np.float32) * (keys[:, None] % 5 + 1)).ok()
    st, before = pull.pull(keys)
    assert st.ok()
    scan = S.ForEachHandler(cl.client, sid, hw)
    for bad in ({"type": "rotate"}, {"type": "scale", "section": 7}, {"type": "clip"}):
        assert scan.for_each(json.dumps(bad))[0].code() == StatusCode.INVALID_CONFIG
    st, r = scan.for_each(json.dumps({"type": "scale", "factor": 0.5}))
    assert st.ok() and r["count"] == 2000                                   # every key once, not once per replica
    assert abs(r["sum"] - 0.5 * float(before.sum())) < 1e-3 * abs(before.sum())
    for _ in range(6):                                                      # reads pick a replica at random
        st, rows = pull.pull(keys)
        assert st.ok() and np.array_equal(rows, np.float32(0.5) * before)
    lim = float(np.abs(before).max()) * 0.25
    st, r = scan.for_each(json.dumps({"type": "clip", "limit": lim}))
    changed = np.abs(np.float32(0.5) * before).max(axis=1) > np.float32(lim)
    assert st.ok() and r["count"] == int(changed.sum()) and r["max_abs"] <= lim * (1 + 1e-6)
    # the accumulator slot is a section of its own: reset it and see the reading scan agree
    st, r = scan.for_each(json.dumps({"type": "fill", "section": 1, "value": 0.25}))
    assert st.ok() and r["count"] == 2000
    st, d = S.ForEachHandler(cl.client, sid, h["for_each"]).for_each(json.dumps({"section": 1}))
    assert st.ok() and d["count"] == 2000 and abs(d["sum"] - 0.25 * 2000 * DIM) < 1e-3 and abs(d["max_abs"] - 0.25) < 1e-7
    st, r = scan.for_each(json.dumps({"type": "fill", "section": 1, "value": 0.25}))
    assert st.ok() and r["count"] == 0                                      # nothing left to change


def test_modulo_partition_places_keys_by_their_value_and_survives_a_reshard(cluster3):
    """`partition: modulo` (the custom partitioner of the reference's predictor test family): key k lives in shard
    k mod N, on client and servers alike, before and after a change of the shard count."""
    cl = cluster3
    ids = cl.ids()
    sid, h = make_table(cl, {ids[0]: [0], ids[1]: [1, 2], ids[2]: [3]}, cfg=op_cfg(partition="modulo"))
    keys = np.concatenate([np.arange(-50, 0), np.arange(1000)]).astype(np.int64)
    vals = np.ones((len(keys), DIM), np.float32) * (np.abs(keys)[:, None] % 13 + 1)
    assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, vals).ok()
    st, info = cl.client.query_storage_info(sid)
    assert st.ok()
    per_shard = {i.shard_id: i.item_number for i in info}
    assert per_shard == {s: int((np.mod(keys, 4) == s).sum()) for s in range(4)}       # numpy's mod is non-negative too
    pull = S.PullHandler(cl.client, sid, h["pull_ro"])
    st, rows = pull.pull(keys)
    assert st.ok() and np.array_equal(rows, vals)
    assert S.UpdateContextHandler(cl.client, sid, h["update_ctx"]).update_context(
        S.nodes_json({ids[0]: [0, 1], ids[1]: [2, 3], ids[2]: [4, 5]})).ok()
    st, info = cl.client.query_storage_info(sid)
    assert st.ok() and {i.shard_id: i.item_number for i in info} == {s: int((np.mod(keys, 6) == s).sum()) for s in range(6)}
    st, rows = pull.pull(keys, 20000, True)
    assert st.ok() and np.array_equal(rows, vals)
    st, _ = cl.client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0]}, op_cfg(partition="zigzag")))
    assert not st.ok() and "partition" in str(st)


def test_bad_placements_and_arguments_are_refused_before_they_cost_data(cluster3, tmp_path):
    """A placement with a gap, without shards or with a shard listed twice, a dim out of range, a dump into no
    directory or into zero files: each is answered with INVALID_CONFIG and the table is as it was."""
    cl = cluster3
    ids = cl.ids()
    create = lambda nodes, **kw: cl.client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config(nodes, op_cfg(**kw)))[0]
    for nodes in ({}, {ids[0]: []}, {ids[0]: [0, 7]}, {ids[0]: [-1, 0]}, {ids[0]: [0, 1, 1]}):
        assert create(nodes).code() == StatusCode.INVALID_CONFIG, nodes
    for dim in (0, -4, 1 << 40):
        assert create({ids[0]: [0]}, dim=dim).code() == StatusCode.INVALID_CONFIG
    sid, h = make_table(cl, {ids[0]: [0], ids[1]: [1], ids[2]: [2]})
    keys = np.arange(300, dtype=np.int64)
    assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, np.ones((300, DIM), np.float32)).ok()
    upd = S.UpdateContextHandler(cl.client, sid, h["update_ctx"])
    for nodes in ("[]", S.nodes_json({ids[0]: [0, 2]}), S.nodes_json({ids[0]: [0], ids[1]: [0, 3]})):
        assert upd.update_context(nodes).code() == StatusCode.INVALID_CONFIG, nodes
    dump = S.DumpHandler(cl.client, sid, h["dump"])
    assert dump.dump("", 1)[0].code() == StatusCode.INVALID_CONFIG              # would have been files in "/"
    assert dump.dump("?format=binary", 1)[0].code() == StatusCode.INVALID_CONFIG
    for n_files in (0, -3):
        assert dump.dump(str(tmp_path / "d"), n_files)[0].code() == StatusCode.INVALID_CONFIG
    assert S.LoadHandler(cl.client, sid, h["load"]).load("")[0].code() == StatusCode.INVALID_CONFIG
    # nothing of all that touched the table
    st, rows = S.PullHandler(cl.client, sid, h["pull_ro"]).pull(keys)
    assert st.ok() and np.all(rows == 1.0)
    assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, np.ones((300, DIM), np.float32)).ok()
    st, n = dump.dump(str(tmp_path / "d"), 2)
    assert st.ok() and n == 300


@pytest.mark.parametrize("n_lost", [1, 2])
def test_a_restore_that_pauses_writes_leaves_the_new_replica_exact(n_lost):
    """`ServerConfig.restore_pauses_writes`: while replacements copy a table from the live replica the table is closed
    to writes (pushes wait in their handlers and go on afterwards), so every push is on the restored replicas exactly
    once - also pushes to rows that were on their way. With two replacements at once the last one to finish opens
    the table again."""
    cl = Cluster(1 + n_lost)
    try:
        ids = cl.ids()
        sid, h = make_table(cl, {n: [0, 1] for n in ids})                     # every node holds everything
        keys = np.arange(20_000, dtype=np.int64)
        ones = np.ones((len(keys), DIM), np.float32)
        assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, ones).ok()
        stop, applied, bad = threading.Event(), [1], []

        def trainer():
            c = S.Client(cl.master.address())
            assert c.initialize_storage(sid).ok()
            push = S.PushHandler(c, sid, h["push"])
            while not stop.is_set():
                st = push.async_push(keys, ones, 60000)
                if not st.ok():
                    bad.append(str(st))
                    return
                applied[0] += 1

        t = threading.Thread(target=trainer)
        t.start()
        try:
            time.sleep(0.2)
            for s in cl.servers[1:]:
                s.stop()                                                       # the trainer's handler finds out and goes on
            deadline = time.time() + 30
            td = S.TableDescriptor()
            while time.time() < deadline:
                td.from_json_str(S.MasterClient(cl.master.address()).get_context(f"storage/{sid}")[1])
                if all(td.node_status()[n] == 1 for n in ids[1:]):
                    break
                time.sleep(0.05)
            assert all(td.node_status()[n] == 1 for n in ids[1:])
            cfg = S.ServerConfig()
            cfg.restore_pauses_writes = True
            cfg.restore_batch_size = 512                                       # many batches: the copy takes a while
            fresh = [S.Server(cl.master.address(), cfg) for _ in range(n_lost)]
            cl.servers += fresh
            before = applied[0]
            results = [None] * n_lost
            workers = [threading.Thread(target=lambda i=i: results.__setitem__(i, fresh[i].restore_storages())) for i in range(n_lost)]
            [w.start() for w in workers]
            [w.join(120) for w in workers]
            assert all(r is not None and r[0].ok() and r[1] == 1 for r in results), results
            td.from_json_str(S.MasterClient(cl.master.address()).get_context(f"storage/{sid}")[1])
            assert td.status() == 0 and all(td.node_status()[f.node_id()] == 0 for f in fresh)   # NORMAL again, the new nodes RUNNING
            deadline = time.time() + 30
            while time.time() < deadline and applied[0] < before + 3:          # the trainer goes on after the pause
                time.sleep(0.05)
            assert applied[0] >= before + 3, (applied, bad)
        finally:
            stop.set()
            t.join(90)
        assert not bad and not t.is_alive(), bad
        cl.servers[0].stop()                                                   # only the restored replicas answer now
        pull = S.PullHandler(cl.client, sid, h["pull_ro"])
        for _ in range(1 if n_lost == 1 else 8):                               # reads pick a replica at random
            st, rows = pull.pull(keys, 20000, True)
            assert st.ok() and np.all(rows == float(applied[0])), (float(rows.min()), float(rows.max()), applied[0])
    finally:
        cl.close()


def test_buffered_sync_pushes_survive_a_reshard_and_a_replica_restore():
    """Sync pushes wait in the rows' delta section until `store`. Rows that move in between - to the new owners of a
    reshard, to a replacement replica - take their pending delta along, and the store folds it there as well."""
    cl = Cluster(2)
    try:
        ids = cl.ids()
        sid, h = make_table(cl, {ids[0]: [0, 1], ids[1]: [0, 1]}, cfg=op_cfg(sync=True))
        keys = np.arange(600, dtype=np.int64)
        push, pull = S.PushHandler(cl.client, sid, h["push"]), S.PullHandler(cl.client, sid, h["pull_ro"])
        assert push.async_push(keys, np.ones((600, DIM), np.float32)).ok()
        assert push.sync_push(keys, 2 * np.ones((600, DIM), np.float32)).ok()          # buffered on both replicas
        # a reshard to three shards moves most rows
        assert S.UpdateContextHandler(cl.client, sid, h["update_ctx"]).update_context(
            S.nodes_json({ids[0]: [0, 1, 2], ids[1]: [0, 1, 2]})).ok()
        assert np.all(pull.pull(keys)[1] == 1.0)                                       # still buffered
        # one replica is lost and replaced
        cl.servers[1].stop()
        td = S.TableDescriptor()
        for _ in range(100):
            assert pull.pull(keys, 20000, True)[0].ok()
            td.from_json_str(S.MasterClient(cl.master.address()).get_context(f"storage/{sid}")[1])
            if td.node_status()[ids[1]] == 1:
                break
        fresh = S.Server(cl.master.address())
        cl.servers.append(fresh)
        st, n = fresh.restore_storages()
        assert st.ok() and n == 1, st
        assert push.store(20000).ok()
        for _ in range(10):                                                            # either replica
            st, rows = pull.pull(keys, 20000, True)
            assert st.ok() and np.all(rows == 3.0), np.unique(rows)
    finally:
        cl.close()


def test_an_operator_can_abort_a_reshard_that_its_client_left_unfinished(cluster3):
    """A client that dies after publishing the target placement leaves the table in RESHARD: reads go on, writes
    wait. `Controller.purge_table` (`psb_node ctl purge SID`) drops the unfinished update; writes resume."""
    cl = cluster3
    ids = cl.ids()
    sid, h = make_table(cl, {ids[0]: [0], ids[1]: [1]})
    keys = np.arange(400, dtype=np.int64)
    ones = np.ones((400, DIM), np.float32)
    push, pull = S.PushHandler(cl.client, sid, h["push"]), S.PullHandler(cl.client, sid, h["pull_ro"])
    assert push.async_push(keys, ones).ok()
    # what the first step of update_context publishes, and then nothing more (the client is gone)
    m = S.MasterClient(cl.master.address())
    td = S.TableDescriptor()
    assert td.from_json_str(m.get_context(f"storage/{sid}")[1])
    assert td.create_update_info(S.nodes_json({ids[0]: [0], ids[1]: [1], ids[2]: [2]})).ok()
    assert m.set_context(f"storage/{sid}", td.to_json_str()).ok() and td.status() == 1
    assert cl.client.pull_context(sid).ok() and cl.client.notify_ctx_update(sid).ok()   # ... and hands to the servers
    st = push.async_push(keys, ones, 1500)
    assert st.code() in (StatusCode.OUT_OF_MEMORY, StatusCode.TIMEOUT), st           # writes wait for the reshard to end
    st, rows = pull.pull(keys, 20000, True)
    assert st.ok() and np.all(rows == 1.0)                                          # reads go on
    ctl = S.Controller(cl.master.address())
    assert ctl.purge_table(sid).ok()
    assert td.from_json_str(m.get_context(f"storage/{sid}")[1]) and td.status() == 0
    assert push.async_push(keys, ones, 20000).ok()
    st, rows = pull.pull(keys, 20000, True)
    assert st.ok() and np.all(rows == 2.0)
    assert ctl.purge_table(4242).code() == StatusCode.INVALID_ID
    # the same way out for a table that a restore with the write pause left closed (status LOADING) when it died
    ctx = json.loads(m.get_context(f"storage/{sid}")[1])
    ctx["status"], ctx["version"] = 2, ctx["version"] + 1
    assert m.set_context(f"storage/{sid}", json.dumps(ctx)).ok()
    assert cl.client.pull_context(sid).ok() and cl.client.notify_ctx_update(sid).ok()
    st = push.async_push(keys, ones, 1500)
    assert st.code() in (StatusCode.OUT_OF_MEMORY, StatusCode.TIMEOUT), st
    assert ctl.purge_table(sid).ok()
    assert td.from_json_str(m.get_context(f"storage/{sid}")[1]) and td.status() == 0
    assert push.async_push(keys, ones, 20000).ok()


def test_dense_ids_and_sizes_that_would_land_on_another_values_keys_are_refused(cluster3):
    """A dense key is (id << 24) | slice. An id of more than 40 bits or a value of more than 2^24 slices would alias
    another value's slices (it used to, silently): both are INVALID_CONFIG now; ids below zero are fine."""
    cl = cluster3
    st, dsid = cl.client.create_storage(S.LIB, "DenseTableStorageOperator", S.storage_config(uneven(cl.ids()), op_cfg(dim=5)))
    assert st.ok()
    _, hp = cl.client.register_handler("pull", S.LIB, "DenseTablePullOperator", "{}", dsid)
    _, hq = cl.client.register_handler("push", S.LIB, "DenseTablePushOperator", "{}", dsid)
    pull, push = S.PullHandler(cl.client, dsid, hp), S.PushHandler(cl.client, dsid, hq)
    v = np.arange(1, 14, dtype=np.float32)
    for tid in (0, 7, -5, (1 << 39) - 1, -(1 << 39) + 1):
        assert push.push_dense(tid, v + tid % 3).ok()
    for tid in (0, 7, -5, (1 << 39) - 1, -(1 << 39) + 1):
        st, back = pull.pull_dense(tid, v.size)
        assert st.ok() and np.array_equal(back, v + tid % 3), tid           # five values, none on another's keys
    for tid in (1 << 39, 1 << 40, -(1 << 39), -(1 << 62)):
        assert push.push_dense(tid, v).code() == StatusCode.INVALID_CONFIG
        assert pull.pull_dense(tid, v.size)[0].code() == StatusCode.INVALID_CONFIG
    assert pull.pull_dense(3, 5 * (1 << 24) + 1)[0].code() == StatusCode.INVALID_CONFIG
    assert pull.pull_dense(0, v.size)[0].ok()


def test_restore_from_dump_when_no_replica(tmp_path):
    cl = Cluster(2)
    try:
        ids = cl.ids()
        sid, h = make_table(cl, {ids[0]: [0], ids[1]: [1]})
        keys = np.arange(1000, dtype=np.int64)
        vals = np.ones((1000, DIM), np.float32) * 3
        assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, vals).ok()
        uri = str(tmp_path / "ckpt")
        assert S.DumpHandler(cl.client, sid, h["dump"]).dump(uri, 1)[0].ok()
        assert cl.client.set_table_uri(sid, uri).ok()
        cl.servers[1].stop()
        pull = S.PullHandler(cl.client, sid, h["pull_ro"])
        st, _ = pull.pull(keys, 3000, True)
        assert st.code() in (StatusCode.NO_REPLICA, StatusCode.TIMEOUT)     # single replica: nothing to fail over to
        fresh = S.Server(cl.master.address())
        cl.servers.append(fresh)
        st, n = fresh.restore_storages()
        assert st.ok() and n == 1, st
        st, rows = pull.pull(keys, 20000, True)
        assert st.ok() and np.array_equal(rows, vals)
    finally:
        cl.close()


def test_memory_limit_backpressure(cluster3):
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()), cfg=op_cfg(dim=64))
    push = S.PushHandler(cl.client, sid, h["push"])
    for s in cl.servers:
        assert s.set_memory_limit(sid, 32 * 1024).ok()
    st = None
    for i in range(50):
        keys = np.arange(i * 500, (i + 1) * 500, dtype=np.int64)
        st = push.async_push(keys, np.ones((500, 64), np.float32), 1000)
        if not st.ok():
            break
    assert st.code() in (StatusCode.OUT_OF_MEMORY, StatusCode.TIMEOUT)
    ok, healthy, used, _ = None, None, None, None
    flags = [cl.client.query_memory_info(n)[1] for n in cl.ids()]
    assert not all(flags)


def test_monitor_thread_brings_a_table_back_after_rows_were_erased():
    """report_interval also drives the memory monitor: a table that refused new rows takes them again once an
    erase_if made room, without anybody touching the health flag."""
    master = S.Master()
    cfg = S.ServerConfig()
    cfg.report_interval_s = 1
    server = S.Server(master.address(), cfg)
    try:
        client = S.Client(master.address())
        sid, h = make_table(type("C", (), {"client": client})(), {server.node_id(): [0, 1]}, cfg=op_cfg(dim=64))
        assert server.set_memory_limit(sid, 96 * 1024).ok()               # rows and index both count
        push = S.PushHandler(client, sid, h["push"])
        st, pushed = None, 0
        for i in range(50):
            keys = np.arange(i * 100, (i + 1) * 100, dtype=np.int64)
            st = push.async_push(keys, np.ones((100, 64), np.float32), 500)
            if not st.ok():
                break
            pushed += 100
        assert st.code() in (StatusCode.OUT_OF_MEMORY, StatusCode.TIMEOUT) and pushed > 0
        assert not client.query_memory_info(server.node_id())[1]
        # three quarters of the keys go: room for the items that the last accepted push had to park, and to spare
        for carried in ({"type": "key_mod", "mod": 2, "rem": 0}, {"type": "key_mod", "mod": 4, "rem": 1}):
            st, erased = S.EraseIfHandler(client, sid, h["erase_if"]).erase_if(json.dumps(carried))
            assert st.ok() and erased > 0
        deadline = time.time() + 10
        while time.time() < deadline and not client.query_memory_info(server.node_id())[1]:
            time.sleep(0.1)
        assert client.query_memory_info(server.node_id())[1]
        fresh = np.arange(10**6, 10**6 + 20, dtype=np.int64)
        assert push.async_push(fresh, np.ones((20, 64), np.float32), 5000).ok()
    finally:
        server.stop()
        master.stop()


def test_scale_out_under_memory_pressure_applies_every_push_exactly_once():
    """A table fills its node: the push that hits the limit is taken as a whole (what finds no row is parked), later
    pushes are refused up front and their client waits; an operator moves a shard to a new node; the parked items
    travel with the shard, the waiting client goes on, and every gradient counts exactly once."""
    master = S.Master()
    a = S.Server(master.address())
    servers = [a]
    try:
        client = S.Client(master.address())
        sid, h = make_table(type("C", (), {"client": client})(), {a.node_id(): [0, 1]}, cfg=op_cfg(memory_limit=256 * 1024))   # rows + index of both shards need 384 KiB, of one shard 192 KiB
        keys = np.arange(6000, dtype=np.int64)
        ones = np.ones((6000, DIM), np.float32)
        done = []

        def trainer():
            push = S.PushHandler(client, sid, h["push"])
            for _ in range(3):
                done.append(push.async_push(keys, ones, 60000))

        t = threading.Thread(target=trainer)
        t.start()
        deadline = time.time() + 20
        while time.time() < deadline and client.query_memory_info(a.node_id())[1]:
            time.sleep(0.02)
        assert not client.query_memory_info(a.node_id())[1]            # the node is full, the trainer is waiting
        assert a.storage_size(sid) < 6000
        b = S.Server(master.address())
        servers.append(b)
        admin = S.Client(master.address())
        assert admin.initialize_storage(sid).ok()
        st = S.UpdateContextHandler(admin, sid, h["update_ctx"]).update_context(S.nodes_json({a.node_id(): [0], b.node_id(): [1]}))
        assert st.ok(), st
        t.join(60)
        assert not t.is_alive() and len(done) == 3 and all(s.ok() for s in done), done
        st, rows = S.PullHandler(admin, sid, h["pull_ro"]).pull(keys, 20000, True)
        assert st.ok() and np.array_equal(rows, 3 * ones), (rows[:, 0].min(), rows[:, 0].max())
        assert a.storage_size(sid) + b.storage_size(sid) == 6000
    finally:
        for s in servers:
            s.stop()
        master.stop()


def test_controller_placement_resize_and_introspection(tmp_path):
    cl = Cluster(4)
    try:
        ctl = S.Controller(cl.master.address())
        st, nodes = ctl.load_nodes()
        assert st.ok() and sorted(nodes) == sorted(cl.ids())
        st, sid = ctl.create_table("ctr_emb", S.LIB, "SparseTableStorageOperator", json.dumps(op_cfg()), 8, 2, S.standard_ops())
        assert st.ok(), st
        client = ctl.client()
        st, hid = client.handler_by_key(sid, "push")
        push = S.PushHandler(client, sid, hid)
        pull = S.PullHandler(client, sid, client.handler_by_key(sid, "pull_ro")[1])
        keys = np.arange(4000, dtype=np.int64)
        vals = np.ones((4000, DIM), np.float32) * (keys[:, None] % 5)
        assert push.async_push(keys, vals).ok()
        table = json.loads(ctl.gen_table_json(sid)[1])
        per_node = {}
        for n in table["context"]["nodes"]:
            per_node[n["g_rank"]] = len(n["shard_list"])
        assert sum(per_node.values()) == 16 and max(per_node.values()) - min(per_node.values()) <= 1   # least-loaded placement
        assert sum(s["item_number"] for s in table["shards"]) == 8000                                     # 2 replicas
        assert ctl.update_table_shard(sid, 12).ok()
        assert np.array_equal(pull.pull(keys)[1], vals)
        assert ctl.update_table_replica(sid, 1).ok()
        table = json.loads(ctl.gen_table_json(sid)[1])
        assert sum(s["item_number"] for s in table["shards"]) == 4000 and len(table["shards"]) == 12
        assert ctl.balance_table(sid).ok()
        assert np.array_equal(pull.pull(keys)[1], vals)
        # scale out: a new server joins, every new node gets 2 new shards
        extra = S.Server(cl.master.address())
        cl.servers.append(extra)
        assert ctl.expand_storage_nodes(sid, [extra.node_id()], 2).ok()
        table = json.loads(ctl.gen_table_json(sid)[1])
        assert len(table["shards"]) == 14 and extra.storage_size(sid) > 0
        assert np.array_equal(pull.pull(keys)[1], vals)
        nodes_view = json.loads(ctl.show_nodes()[1])
        assert len(nodes_view) == 5 and all(n["alive"] for n in nodes_view)
        # the data verbs of the command line, from Python
        st, stats = ctl.table_stats(sid)
        assert st.ok() and json.loads(stats)["count"] == 4000
        st, n = ctl.dump_table(sid, str(tmp_path / "ctl_dump"), 2)
        assert st.ok() and n == 4000
        st, sid_copy = ctl.create_table("copy", S.LIB, "SparseTableStorageOperator", json.dumps(op_cfg()), 3, 1, S.standard_ops())
        assert st.ok(), st
        st, n = ctl.load_table(sid_copy, str(tmp_path / "ctl_dump"))
        assert st.ok() and n == 4000
        assert json.loads(ctl.table_stats(sid_copy)[1])["count"] == 4000
        st, n = ctl.erase_from_table(sid_copy, json.dumps({"type": "key_mod", "mod": 4, "rem": 1}))
        assert st.ok() and n == 1000 and ctl.delete_table(sid_copy).ok()
        # a storage without a table object is cleaned up
        st, orphan = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({cl.ids()[0]: [0]}, op_cfg()))
        st, removed = ctl.clean_unused_storage()
        assert st.ok() and removed == 1
        assert ctl.shutdown_node(extra.node_id()).ok()
        for _ in range(100):
            if extra.exited():
                break
            time.sleep(0.05)
        assert extra.exited()
        assert ctl.delete_table(sid).ok()
    finally:
        cl.close()


def test_predictor_sync_udf_and_native_ps(tmp_path, cluster3):
    cl = cluster3
    ids = cl.ids()
    cfg = op_cfg(optimizer="sgd", lr=1.0)
    trainer, ht = make_table(cl, {ids[0]: [0], ids[1]: [1]}, cfg=cfg)
    predictor, hp = make_table(cl, {ids[2]: [0, 1, 2]}, cfg=cfg)
    for s in cl.servers[:2]:
        assert s.enable_sync(trainer).ok()
    push = S.PushHandler(cl.client, trainer, ht["push"])
    keys = np.arange(500, dtype=np.int64)
    assert push.async_push(keys, -np.ones((500, DIM), np.float32)).ok()
    sync = S.SyncHandler(cl.client, predictor, hp["sync"])
    total = 0
    for s in cl.servers[:2]:
        st, n = s.push_sync_table(trainer, sync)
        assert st.ok(), st
        total += n
    assert total == 500
    ppull = S.PullHandler(cl.client, predictor, hp["pull_ro"])
    assert np.all(ppull.pull(keys)[1] == 1.0)
    # only what changed since the last round travels
    assert push.async_push(keys[:7], -np.ones((7, DIM), np.float32)).ok()
    assert sum(s.push_sync_table(trainer, sync)[1] for s in cl.servers[:2]) == 7
    assert np.all(ppull.pull(keys[:7])[1] == 2.0)
    assert sum(s.push_sync_table(trainer, sync)[1] for s in cl.servers[:2]) == 0
    # rows that a writing scan changed are part of the next increment, rows that it left alone are not
    st, hw = cl.client.register_handler("for_each_write", S.LIB, "ForEachWriteOperator", "{}", trainer)
    assert st.ok(), st
    st, r = S.ForEachHandler(cl.client, trainer, hw).for_each(json.dumps({"type": "clip", "limit": 1.5}))
    assert st.ok() and r["count"] == 7
    assert sum(s.push_sync_table(trainer, sync)[1] for s in cl.servers[:2]) == 7
    assert np.all(ppull.pull(keys[:7])[1] == 1.5) and np.all(ppull.pull(keys[7:])[1] == 1.0)
    st, r = S.ForEachHandler(cl.client, trainer, hw).for_each(json.dumps({"type": "fill", "value": 2.0}))
    assert st.ok() and r["count"] == 500 and push.async_push(keys[:7], np.zeros((7, DIM), np.float32)).ok()
    assert sum(s.push_sync_table(trainer, sync)[1] for s in cl.servers[:2]) == 500
    # UDF: a Python function registered on the servers
    S.register_udf("count_items", lambda sid, items, param: f"{items}:{param.decode()}".encode())
    st, hid = cl.client.register_handler("udf", S.LIB, "UDFOperator", json.dumps({"function": "count_items"}), trainer)
    st, results = S.UDFHandler(cl.client, trainer, hid).call(b"hello")
    assert st.ok() and sorted(int(r.split(b":")[0]) for _, r in results) == sorted(s.storage_size(trainer) for s in cl.servers[:2])
    # request building split from sending: a request built before a context change is refused, a fresh one passes
    udf = S.UDFHandler(cl.client, trainer, hid)
    st, req = udf.generate_request(b"x")
    assert st.ok() and sorted(req.nodes()) == sorted(ids[:2])
    st, results = udf.send_request(req)
    assert st.ok() and len(results) == 2
    assert S.UpdateContextHandler(cl.client, trainer, ht["update_ctx"]).update_context(
        S.nodes_json({ids[0]: [1], ids[1]: [0]})).ok()                     # a reshard: new context version
    st, _ = udf.send_request(req)
    assert st.code() == StatusCode.SERVER_TOO_NEW_CTX
    st, req = udf.generate_request(b"y")
    assert udf.send_request(req)[0].ok()
    # NativePS: in-process load of a distributed dump + pull
    uri = str(tmp_path / "serving")
    assert S.DumpHandler(cl.client, trainer, ht["dump"]).dump(uri, 2)[0].ok()
    nps = S.NativePS()
    st, nsid = nps.create_storage(S.LIB, "SparseTableStorageOperator", json.dumps(cfg), 3)
    _, lh = nps.register_handler(nsid, "load", S.LIB, "LoadOperator", "{}")
    _, ph = nps.register_handler(nsid, "pull", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}))
    st, n = S.NativeLoadHandler(nps, nsid, lh).load(uri, 4)
    assert st.ok() and n == 500 and nps.size(nsid) == 500
    st, rows = S.NativePullHandler(nps, nsid, ph).pull(keys, DIM)
    assert st.ok() and np.all(rows == 2.0)
    native = S.NativePullHandler(nps, nsid, ph)
    assert native.dim() == DIM and native.pull(keys)[1].shape == (500, DIM)                 # the table's width by default
    assert native.pull(keys, DIM - 1)[0].code() == StatusCode.INVALID_CONFIG                # not a short buffer written over


def test_common_pieces():
    wire, body, sid, hid, ver, uver, typ = C.message_round_trip(b"payload", 3, 4, 5, 6, 10)
    assert body == b"payload" and (sid, hid, ver, uver, typ) == (3, 4, 5, 6, 10) and len(wire) == 7 + 20
    assert C.request_type_name(10) == "OP_PULL" and C.request_type_name(23) == "OP_COORDINATED_RESTORE_ITERATE"
    r = C.archive_round_trip(-7, 2.5, "héllo", [1, 2, 3], ["a", "bc"])
    assert r[:5] == (-7, 2.5, "héllo", [1, 2, 3], ["a", "bc"]) and r[5] == 3 and r[6] == "full" and r[7]
    data = bytes(range(256)) * 100
    for algo in ("", "zstd", "lz4", "snappy"):
        st, back, packed = C.compress_round_trip(algo, data)
        assert st.ok() and back == data and (algo == "" or packed < len(data))
    assert not C.compress_round_trip("bogus", b"x")[0].ok()
    v = list(np.random.default_rng(0).standard_normal(100))
    assert C.heap_sort(v) == sorted(v)
    # request coalescing: two threads finish, the second one claims both slots
    tr = C.ThreadReduce()
    tr.add(0); tr.add(1)
    assert tr.reduce(0, 2) == 0
    assert tr.reduce(1, 2) == 0b11
    tb = C.ThreadBcast()
    t = threading.Thread(target=lambda: tb.wait(0))
    t.start()
    tb.notify(0b11, 1)
    t.join(5)
    assert not t.is_alive()
    model = {"name": "m", "type": "ctr", "version": "1", "status": 0, "submodels": [
        {"name": "sub", "type": "", "version": "", "status": 0, "submodels": [], "tables": [
            {"table_name": "t2", "table_uri": "", "lib_name": "psb", "init_method": 0, "shard_num": 2, "replica_num": 1, "storage_id": 9,
             "storage_op": {"key": "storage", "lib_name": "psb", "op_name": "S", "config_str": "{}", "handler_id": -1},
             "ops": [{"key": "pull", "lib_name": "psb", "op_name": "P", "config_str": "{}", "handler_id": 3}]}]}],
        "tables": []}
    back = json.loads(C.model_round_trip(json.dumps(model)))
    assert back["n_tables"] == 1 and back["n_operators"] == 1 and back["submodels"][0]["tables"][0]["storage_id"] == 9


def test_table_descriptor_state_machine():
    td = S.TableDescriptor()
    assert td.set_nodes(S.nodes_json({0: [0, 1], 1: [1, 2], 2: [2, 0]})).ok()
    assert td.global_shard_num() == 3 and td.shards()[1] == [0, 1]
    assert td.update_node_status({0, 2}) and td.node_status()[1] == 1
    assert td.shards()[1] == [0]
    picks = {td.pick_one_replica(2) for _ in range(50)}
    assert picks == {2}
    v = td.version
    assert td.try_to_replace_one_dead_node(7) and td.node_status() == {0: 0, 7: 2, 2: 0} and td.version == v + 1
    assert td.pick_one_replica(1) == 0            # LOADING nodes are not picked
    assert td.set_node_status_to_running(7) and td.node_status()[7] == 0
    uv = td.update_version
    assert td.create_update_info(S.nodes_json({0: [0], 2: [1], 7: [2], 9: [3]})).ok()
    assert td.status() == 1 and td.update_version == uv + 1
    td2 = S.TableDescriptor()
    assert td2.from_json_str(td.to_json_str())
    assert td2.to_json_str() == td.to_json_str()
    assert not td2.from_json_str(td.to_json_str(), True)      # not newer: left alone
    td.apply_update()
    assert td.global_shard_num() == 4 and td.update_version == uv + 2
    assert td2.from_json_str(td.to_json_str(), True)


def test_pull_requests_of_threads_are_merged(cluster3):
    """Small pulls of handlers on different threads travel as one message per node and every thread still
    gets exactly its own rows (ThreadReduce / ThreadBcast coalescing)."""
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()))
    push = S.PushHandler(cl.client, sid, h["push"])
    keys = np.arange(4000, dtype=np.int64)
    g = (keys[:, None] * np.ones((1, DIM))).astype(np.float32)
    assert push.async_push(keys, g).ok()
    group = S.PullGroup()
    T = 4
    hs = [S.PullHandler(cl.client, sid, h["pull_ro"]) for _ in range(T)]
    assert [x.join_group(group) for x in hs] == list(range(T))
    rng = np.random.default_rng(0)
    batches = [[rng.integers(0, 4000, size=300).astype(np.int64) for _ in range(30)] for _ in range(T)]
    bad = []

    def work(t):
        for b in batches[t]:
            st, rows = hs[t].pull(b)
            if not (st.ok() and np.array_equal(rows, g[b])):
                bad.append((t, str(st)))

    ts = [threading.Thread(target=work, args=(t,)) for t in range(T)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert not bad and not any(t.is_alive() for t in ts)
    assert group.merged_requests() == T * 30
    assert group.merged_sends() < group.merged_requests()      # some requests did share a message


def test_push_requests_of_threads_are_merged(cluster3):
    """Small pushes of handlers on different threads share messages; every gradient is applied exactly once."""
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()))
    group = S.PushGroup()
    T = 4
    hs = [S.PushHandler(cl.client, sid, h["push"]) for _ in range(T)]
    assert [x.join_group(group) for x in hs] == list(range(T))
    rng = np.random.default_rng(1)
    batches = [[rng.integers(0, 3000, size=200).astype(np.int64) for _ in range(25)] for _ in range(T)]
    bad = []

    def work(t):
        for b in batches[t]:
            st = hs[t].async_push(b, np.ones((len(b), DIM), dtype=np.float32))
            if not st.ok():
                bad.append((t, str(st)))

    ts = [threading.Thread(target=work, args=(t,)) for t in range(T)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert not bad and not any(t.is_alive() for t in ts)
    assert group.merged_requests() == T * 25 and group.merged_sends() < group.merged_requests()
    counts = np.bincount(np.concatenate([b for bs in batches for b in bs]), minlength=3000).astype(np.float32)
    keys = np.arange(3000, dtype=np.int64)
    st, rows = S.PullHandler(cl.client, sid, h["pull_ro"]).pull(keys)
    assert st.ok() and np.array_equal(rows, counts[:, None] * np.ones((1, DIM), dtype=np.float32))


@pytest.mark.parametrize("cap", [1, 2])
def test_max_request_merge_num_caps_what_one_message_carries(cluster3, cap):
    """`max_request_merge_num` in the operator config: 1 switches the coalescing off (one message per request), 2 lets
    at most two requests share a message; results and exactly-once application are unaffected."""
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()))
    st, h_pull = cl.client.register_handler("pull_capped", S.LIB, "SparseTablePullOperator",
                                            json.dumps({"read_only": True, "max_request_merge_num": cap}), sid)
    assert st.ok()
    st, h_push = cl.client.register_handler("push_capped", S.LIB, "SparseTablePushOperator",
                                            json.dumps({"max_request_merge_num": cap}), sid)
    assert st.ok()
    T = 4
    pgroup, qgroup = S.PullGroup(), S.PushGroup()
    pulls = [S.PullHandler(cl.client, sid, h_pull) for _ in range(T)]
    pushes = [S.PushHandler(cl.client, sid, h_push) for _ in range(T)]
    assert [x.join_group(pgroup) for x in pulls] == list(range(T)) and [x.join_group(qgroup) for x in pushes] == list(range(T))
    rng = np.random.default_rng(2)
    batches = [[rng.integers(0, 2000, size=150).astype(np.int64) for _ in range(20)] for _ in range(T)]
    bad = []

    def work(t):
        for b in batches[t]:
            if not pushes[t].async_push(b, np.ones((len(b), DIM), dtype=np.float32)).ok():
                bad.append(("push", t))
            st, rows = pulls[t].pull(b)
            if not st.ok() or rows.shape != (len(b), DIM):
                bad.append(("pull", t))

    ts = [threading.Thread(target=work, args=(t,)) for t in range(T)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert not bad and not any(t.is_alive() for t in ts)
    for g in (pgroup, qgroup):
        assert g.merged_requests() == T * 20
        assert g.merged_sends() * cap >= g.merged_requests()           # no message carried more than `cap` requests
        if cap == 1:
            assert g.merged_sends() == g.merged_requests()
    counts = np.bincount(np.concatenate([b for bs in batches for b in bs]), minlength=2000).astype(np.float32)
    st, rows = S.PullHandler(cl.client, sid, h["pull_ro"]).pull(np.arange(2000, dtype=np.int64))
    assert st.ok() and np.array_equal(rows, counts[:, None] * np.ones((1, DIM), dtype=np.float32))


def test_operator_config_keys_of_the_reference_are_understood(cluster3):
    cl = cluster3
    cfg = op_cfg()
    cfg["pool_hash_map"] = {"expected_max_items": 50000, "grow_ratio": 2.0}
    sid, h = make_table(cl, uneven(cl.ids()), cfg=cfg)
    st, hid = cl.client.register_handler("pull_random", S.LIB, "SparseTablePullOperator",
                                         json.dumps({"read_only": True, "node_selection": "random"}), sid)
    assert st.ok()
    st, _ = cl.client.register_handler("pull_nearest", S.LIB, "SparseTablePullOperator",
                                       json.dumps({"node_selection": "nearest"}), sid)
    assert not st.ok() and "node_selection" in str(st)
    # the refused registration left nothing behind: the table still works with the handlers it had
    keys = np.arange(100, dtype=np.int64)
    assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, np.ones((100, DIM), np.float32)).ok()
    st, rows = S.PullHandler(cl.client, sid, hid).pull(keys)
    assert st.ok() and np.all(rows == 1.0)


def test_runtime_log_lines_reach_python_logging(caplog):
    """The native runtime logs its life-cycle events (a server joining, storages created, a node found dead, a restore
    and its source); `service.log_to_python` hands the lines to the logging module."""
    import logging
    S.set_log_level("info")
    S.log_to_python("psb_test")
    try:
        with caplog.at_level(logging.INFO, logger="psb_test"):
            cl = Cluster(2)
            try:
                ids = cl.ids()
                sid, h = make_table(cl, {ids[0]: [0, 1], ids[1]: [0, 1]})
                keys = np.arange(50, dtype=np.int64)
                assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, np.ones((50, DIM), np.float32)).ok()
                cl.servers[1].stop()
                pull = S.PullHandler(cl.client, sid, h["pull_ro"])
                for _ in range(20):
                    assert pull.pull(keys, 20000, True)[0].ok()
                fresh = S.Server(cl.master.address())
                cl.servers.append(fresh)
                st, n = fresh.restore_storages()
                assert st.ok() and n == 1
            finally:
                cl.close()
        text = "\n".join(r.getMessage() for r in caplog.records)
        assert f"pserver node {ids[0]} serves c2s" in text
        assert f"storage {sid} created on node {ids[0]}" in text
        assert "marked DEAD" in text and f"takes the place of dead node {ids[1]}" in text
        assert f"storage {sid}: restored from replica, 50 items" in text
        assert any(r.levelno == logging.WARNING for r in caplog.records)
    finally:
        C.set_log_sink(None)
        S.set_log_level("warning")


def test_a_server_that_lost_its_master_session_registers_again_unless_it_was_declared_dead():
    cfg = S.ServerConfig()
    cfg.session_check_ms = 100
    master = S.Master()
    servers = [S.Server(master.address(), cfg) for _ in range(2)]
    try:
        client = S.Client(master.address())
        ids = [s.node_id() for s in servers]
        sid, h = make_table(type("C", (), {"client": client})(), {ids[0]: [0, 1], ids[1]: [0, 1]})
        keys = np.arange(200, dtype=np.int64)
        assert S.PushHandler(client, sid, h["push"]).async_push(keys, np.ones((200, DIM), np.float32)).ok()

        def listed():
            st, nodes = client.get_pserver_list()
            return sorted(nodes) if st.ok() else None

        # a dropped connection alone: the node is back in the registry within a few checks, nobody noticed
        servers[0].drop_master_session()
        deadline = time.time() + 5
        while time.time() < deadline and listed() != sorted(ids):
            time.sleep(0.02)
        assert listed() == sorted(ids)
        # the same fault, but this time a client sees the gap and publishes the node as DEAD before it is back:
        # the node must stay out (a replacement will take its place under a new id)
        slow = S.ServerConfig()
        slow.session_check_ms = 1500
        late = S.Server(master.address(), slow)
        servers.append(late)
        sid2, h2 = make_table(type("C", (), {"client": client})(), {late.node_id(): [0], ids[1]: [0]})
        late.drop_master_session()
        pull = S.PullHandler(client, sid2, h2["pull_ro"])
        deadline = time.time() + 1.2
        while time.time() < deadline:
            assert pull.pull(keys, 5000, True)[0].ok()          # reads go on from the other replica; the gap gets noticed
        td = S.TableDescriptor()
        td.from_json_str(S.MasterClient(master.address()).get_context(f"storage/{sid2}")[1])
        assert td.node_status()[late.node_id()] == 1               # DEAD in the published context
        stale = S.Client(master.address())                          # a client that will not hear of the change by itself
        time.sleep(2.0)                                             # several checks of the late server pass
        assert late.node_id() not in (listed() or [])
        # data requests that still reach the replaced node are turned away with the status that makes clients refresh
        assert stale.initialize_storage(sid2).ok()
        for _ in range(10):
            assert S.PullHandler(stale, sid2, h2["pull_ro"]).pull(keys, 5000, True)[0].ok()
    finally:
        for s in servers:
            s.stop()
        master.stop()


def test_calls_in_flight_overlap_and_are_waited_for(cluster3):
    """start(...) / wait(): pushes and pulls of several handlers are in flight together."""
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()))
    keys = np.arange(3000, dtype=np.int64)
    parts = np.array_split(keys, 6)
    pending = [S.start(S.PushHandler(cl.client, sid, h["push"]).async_push, p, np.ones((len(p), DIM), np.float32)) for p in parts]
    assert all(p.wait(30).ok() for p in pending)
    pulls = [S.start(S.PullHandler(cl.client, sid, h["pull_ro"]).pull, p) for p in parts]
    for p, part in zip(pulls, parts):
        st, rows = p.wait(30)
        assert st.ok() and rows.shape == (len(part), DIM) and np.all(rows == 1.0)
    assert all(p.done() for p in pulls)
    bad = S.start(S.PushHandler(cl.client, sid, h["push"]).async_push, keys, np.ones((5, DIM), np.float32))   # wrong shape
    with pytest.raises(ValueError):
        bad.wait(30)


def test_available_server_list_excludes_stopped_nodes(cluster3):
    cl = cluster3
    st, nodes = cl.client.get_available_pserver_list()
    assert st.ok() and sorted(nodes) == sorted(cl.ids())
    cl.servers[2].stop()
    st, nodes = cl.client.get_available_pserver_list(500)
    assert st.ok() and sorted(nodes) == sorted(cl.ids()[:2])


def test_one_way_context_refresh_and_predictor_create(cluster3):
    """require_update_ctx_async tells the servers to re-read a table's context without waiting for them;
    pred_create_storage is the predictor-side name of create_storage."""
    cl = cluster3
    st, sid = cl.client.pred_create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config(uneven(cl.ids()), op_cfg()))
    assert st.ok() and sid >= 0
    before = [s.metrics_text().count("CTX_UPDATE") for s in cl.servers]
    cl.client.require_update_ctx_async(sid)            # returns at once
    deadline = time.time() + 5
    while time.time() < deadline and not all('request_type="c2s_ctx_update"' in s.metrics_text() for s in cl.servers):
        time.sleep(0.02)
    assert all('request_type="c2s_ctx_update"' in s.metrics_text() for s in cl.servers), before
    # the channel is still good for ordinary calls afterwards (the late answers were dropped by the reader)
    st, hid = cl.client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
    assert st.ok() and S.PullHandler(cl.client, sid, hid).pull(np.arange(10, dtype=np.int64))[0].ok()
    cl.client.require_update_ctx_async(12345)          # unknown table: nothing happens


def test_prometheus_metrics_endpoint(cluster3):
    import urllib.request
    from parameter_server_b200.service.metrics import handler_metrics_text, serve_metrics
    cl = cluster3
    sid, h = make_table(cl, uneven(cl.ids()))
    push, pull = S.PushHandler(cl.client, sid, h["push"]), S.PullHandler(cl.client, sid, h["pull_ro"])
    keys = np.arange(500, dtype=np.int64)
    assert push.async_push(keys, np.ones((500, DIM), np.float32)).ok()
    assert pull.pull(keys)[0].ok()
    httpd, port = serve_metrics(cl.servers[0], 0, [sid])
    try:
        text = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
    finally:
        httpd.shutdown()
    node = cl.servers[0].node_id()
    assert f'ps_requests_total{{node_id="{node}",request_type="c2s_pull",storage_id="{sid}"}} 1' in text
    assert f'ps_requests_total{{node_id="{node}",request_type="c2s_async_push",storage_id="{sid}"}} 1' in text
    assert 'ps_request_duration_ms_bucket' in text and 'le="+Inf"' in text and "ps_response_size_bytes" in text
    assert f'ps_storage_items{{node_id="{node}",storage_id="{sid}"}}' in text
    assert "ps_wait_request_count" in handler_metrics_text(pull, "pull")
    assert 'ps_pull_send_request_count{handler="pull"} 1' in handler_metrics_text(pull, "pull")
    assert "ps_pull_send" not in handler_metrics_text(push, "push")


def test_sync_pred_backs_off_and_resumes_after_the_predictor_comes_back():
    """The predictor's only server is down when the sync starts: the pass fails (time-out -> dead node ->
    no replica), the dirty marks stay, the handler backs off; meanwhile a fresh server restores the predictor table
    from its dump, and a later attempt delivers everything."""
    import tempfile
    cl = Cluster(3)
    try:
        ids = cl.ids()
        cfg = op_cfg(optimizer="sgd", lr=1.0)
        trainer, ht = make_table(cl, {ids[0]: [0, 1]}, cfg=cfg)
        predictor, hp = make_table(cl, {ids[2]: [0, 1]}, cfg=cfg)
        assert cl.servers[0].enable_sync(trainer).ok()
        uri = tempfile.mkdtemp(prefix="psb_pred_")
        assert S.DumpHandler(cl.client, predictor, hp["dump"]).dump(uri, 1)[0].ok()   # (empty) image for the restore
        assert cl.client.set_table_uri(predictor, uri).ok()
        keys = np.arange(300, dtype=np.int64)
        assert S.PushHandler(cl.client, trainer, ht["push"]).async_push(keys, -np.ones((300, DIM), np.float32)).ok()
        cl.servers[2].stop()                                     # the predictor's server is gone
        sync = S.SyncHandler(cl.client, predictor, hp["sync"])
        result = {}

        def run_sync():
            result["out"] = sync.sync_pred(cl.servers[0], trainer, max_attempts=8, backoff_scale=0.1)

        th = threading.Thread(target=run_sync)
        th.start()
        time.sleep(0.8)                                          # a few failed passes with back-off
        fresh = S.Server(cl.master.address())
        cl.servers.append(fresh)
        st, n = fresh.restore_storages()
        assert st.ok() and n == 1, st
        th.join(60)
        assert not th.is_alive()
        st, n = result["out"]
        assert st.ok(), st
        assert n >= 300                                          # everything arrived (a failed pass may have re-sent blocks)
        assert sync.metrics()["retries"] >= 1
        st, rows = S.PullHandler(cl.client, predictor, hp["pull_ro"]).pull(keys, 20000, True)
        assert st.ok() and np.all(rows == 1.0)
    finally:
        cl.close()


def test_deleting_a_table_removes_its_image_unless_retained(tmp_path):
    """A table's saved image goes with the table; `pmem_create_storage.retain_dcpmm_data_after_deconstruction` (the
    reference's spelling) or `retain_local_image` keeps it. The index ratios of the reference's storage sections are
    accepted on the same config."""
    cfg = S.ServerConfig()
    cfg.local_image_dir = str(tmp_path / "images")
    master = S.Master()
    server = S.Server(master.address(), cfg)
    client = S.Client(master.address())
    try:
        nid = server.node_id()
        plain = op_cfg()
        plain["google_dense_hash_map"] = {"shrink_ratio": 0.2, "grow_ratio": 0.7, "expected_max_items": 1000}
        kept = op_cfg()
        kept["pmem_create_storage"] = {"storage_id": 7, "retain_dcpmm_data_after_deconstruction": 1}
        sids = []
        for c in (plain, kept):
            st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({nid: [0, 1]}, c))
            assert st.ok(), st
            sids.append(sid)
        st, n = server.save_local_images()
        assert st.ok() and n == 2
        imgs = [tmp_path / "images" / f"node_{nid}" / f"storage_{sid}.img" for sid in sids]
        assert all(p.exists() for p in imgs)
        for sid in sids:
            assert client.delete_storage(sid).ok()
        assert not imgs[0].exists() and imgs[1].exists()
    finally:
        server.stop()
        master.stop()


def test_restore_from_the_hosts_own_image_when_no_replica(tmp_path):
    """No replica, no dump: the replacement server opens the persistent image that the dead node left on this host
    (the role of the reference's persistent-memory pool). An image of another data layout is refused."""
    cfg = S.ServerConfig()
    cfg.local_image_dir = str(tmp_path / "images")
    master = S.Master()
    servers = [S.Server(master.address(), cfg) for _ in range(2)]
    client = S.Client(master.address())
    try:
        ids = [s.node_id() for s in servers]
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0, 1], ids[1]: [2]}, op_cfg()))
        assert st.ok()
        _, hq = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
        _, hp = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
        keys = np.arange(1500, dtype=np.int64)
        vals = np.ones((1500, DIM), np.float32) * (keys[:, None] % 5 + 1)
        assert S.PushHandler(client, sid, hq).async_push(keys, vals).ok()
        for s in servers:
            st, n = s.save_local_images()
            assert st.ok() and n == 1
        import shutil
        src = tmp_path / "images" / f"node_{ids[0]}" / f"storage_{sid}.img"
        kept = tmp_path / "kept.img"
        shutil.copy(src, kept)
        stale = tmp_path / "images" / f"node_{ids[1]}" / "storage_4242.img"   # a table that the master does not know
        shutil.copy(src, stale)
        servers[0].stop()                                           # the node with shards 0 and 1 is gone
        pull = S.PullHandler(client, sid, hp)
        assert not pull.pull(keys, 3000, True)[0].ok()              # nobody holds those shards now
        fresh = S.Server(master.address(), cfg)
        servers.append(fresh)
        st, n = fresh.restore_storages()
        assert st.ok() and n == 1, st
        st, rows = pull.pull(keys, 20000, True)
        assert st.ok() and np.array_equal(rows, vals)
        # housekeeping after the restore: the replaced node's images are used up, the unknown table's image is stale,
        # the live neighbour's image of the current table stays
        assert not src.exists() and not src.parent.exists() and not stale.exists()
        assert (tmp_path / "images" / f"node_{ids[1]}" / f"storage_{sid}.img").exists()
        # a table created anew has another version_uuid: an old image with the same ids must not be opened
        st, sid2 = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({fresh.node_id(): [0]}, op_cfg()))
        assert st.ok()
        src = kept
        dst = tmp_path / "images" / f"node_{fresh.node_id()}" / f"storage_{sid2}.img"
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copy(src, dst)
        fresh.stop()
        last = S.Server(master.address(), cfg)
        servers.append(last)
        st, n = last.restore_storages()
        assert not st.ok()                                          # no replica, foreign image refused, no dump either
        # the same housekeeping from outside a server: what lies in the directory and whose it is
        st, listing = C.list_local_images(str(tmp_path / "images"), master.address())
        assert st.ok()
        states = {(im["node"], im["storage_id"]): im["state"] for im in json.loads(listing)}
        assert states[(fresh.node_id(), sid2)] == "stale"          # copied from another table
        assert states[(ids[1], sid)] == "current" and all(im["records"] > 0 for im in json.loads(listing))
        assert [im["state"] for im in json.loads(C.list_local_images(str(tmp_path / "images"))[1])] == ["unknown"] * len(states)
        (tmp_path / "images" / f"node_{ids[1]}" / "storage_77.img").write_bytes(b"PSBIMG1\0garbage")
        st, n = C.remove_unused_local_images(str(tmp_path / "images"), master.address())
        assert st.ok() and n == 2 and not dst.exists()              # the foreign image and the damaged one go
        assert (tmp_path / "images" / f"node_{ids[1]}" / f"storage_{sid}.img").exists()
        servers[1].stop()                                           # its image is now that of a node that is gone
        for _ in range(100):
            if json.loads(C.list_local_images(str(tmp_path / "images"), master.address())[1])[0]["state"] == "dead_node":
                break
            time.sleep(0.05)
        assert C.remove_unused_local_images(str(tmp_path / "images"), master.address())[1] == 0   # kept for a restore
        assert C.remove_unused_local_images(str(tmp_path / "images"), master.address(), True)[1] == 1
        st, n = last.clean_local_images()
        assert st.ok() and n == 0
    finally:
        for s in servers:
            s.stop()
        master.stop()


def test_server_config_report_restore_wait_and_threaded_load(tmp_path):
    """ServerConfig knobs: the periodic report line, a restore-mode server that waits for a node to die, and a
    load request whose files are read by several threads."""
    cfg = S.ServerConfig()
    cfg.report_interval_s = 1
    cfg.load_thread_num = 3
    master = S.Master()
    servers = [S.Server(master.address(), cfg) for _ in range(2)]
    client = S.Client(master.address())
    try:
        ids = [s.node_id() for s in servers]
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                        S.storage_config({ids[0]: [0, 1, 2], ids[1]: [0, 1, 2]}, op_cfg()))
        assert st.ok()
        h = {}
        for key, op, c in [("push", "SparseTablePushOperator", {}), ("pull_ro", "SparseTablePullOperator", {"read_only": True}),
                           ("dump", "DumpOperator", {}), ("load", "LoadOperator", {"block_size": 50})]:
            st, h[key] = client.register_handler(key, S.LIB, op, json.dumps(c), sid)
            assert st.ok()
        keys = np.arange(3000, dtype=np.int64)
        vals = np.ones((3000, DIM), np.float32) * (keys[:, None] % 3 + 1)
        assert S.PushHandler(client, sid, h["push"]).async_push(keys, vals).ok()
        uri = str(tmp_path / "d")
        st, n = S.DumpHandler(client, sid, h["dump"]).dump(uri, 5)          # several files per node
        assert st.ok() and n == 3000
        assert client.clear_storage(sid).ok()
        st, n = S.LoadHandler(client, sid, h["load"]).load(uri, 8, 30000)   # one wave: a server gets many files at once
        assert st.ok() and n == 3000
        st, rows = S.PullHandler(client, sid, h["pull_ro"]).pull(keys)
        assert st.ok() and np.array_equal(rows, vals)
        line = servers[0].report_line()
        assert line.startswith(f"pserver node={ids[0]} requests=") and f"{sid}:" in line
        time.sleep(1.5)
        assert servers[0].last_report().startswith(f"pserver node={ids[0]}")
        # restore mode with a wait: the replacement starts BEFORE the node dies and still takes over
        rcfg = S.ServerConfig()
        rcfg.restore_wait_timeout_s = 10
        box = {}

        def replacement():
            fresh = S.Server(master.address(), rcfg)
            box["server"] = fresh
            box["out"] = fresh.restore_storages()

        th = threading.Thread(target=replacement)
        th.start()
        time.sleep(0.5)
        servers[1].stop()
        th.join(30)
        assert not th.is_alive()
        st, n = box["out"]
        assert st.ok() and n == 1, st
        servers.append(box["server"])
        assert box["server"].storage_size(sid) == 3000
    finally:
        for s in servers:
            s.stop()
        master.stop()
