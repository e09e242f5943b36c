"""The sync thread of a server: a trainer table whose push operator names follower tables keeps a predictor table
(in another cluster, found through the model registry of that cluster's master) fresh in the background."""
import json
import time

import numpy as np

from parameter_server_b200 import C
from parameter_server_b200 import service as S

DIM = 4
OPT = dict(dim=DIM, optimizer="sgd", lr=1.0, init_range=0.0, sync=True)


def _table(client, nodes, push_cfg):
    st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config(nodes, OPT))
    assert st.ok(), st
    h = {}
    for key, op, cfg in [("pull_ro", "SparseTablePullOperator", {"read_only": True}), ("push", "SparseTablePushOperator", push_cfg),
                         ("sync", "KVSyncOperator", {"block_size": 64}), ("update_ctx", "ShardUpdateContextOperator", {})]:
        st, h[key] = client.register_handler(key, S.LIB, op, json.dumps(cfg), sid)
        assert st.ok(), st
    return sid, h


def _model(name, table_name, sid, handlers):
    ops = [{"key": k, "lib_name": S.LIB, "op_name": "", "config_str": "{}", "handler_id": hid} for k, hid in handlers.items()]
    return {"name": name, "type": "ctr", "version": "1", "status": 0, "submodels": [], "tables": [
        {"table_name": table_name, "table_uri": "", "lib_name": S.LIB, "init_method": 0, "shard_num": 3, "replica_num": 1,
         "storage_id": sid, "storage_op": {"key": "storage", "lib_name": S.LIB, "op_name": "", "config_str": "{}", "handler_id": -1},
         "ops": ops}]}


def _wait(pred, seconds=10.0):
    t0 = time.time()
    while time.time() - t0 < seconds:
        if pred():
            return True
        time.sleep(0.02)
    return False


def test_pushes_on_a_followed_table_reach_the_predictor_cluster():
    tm, pm = S.Master(), S.Master()                       # trainer cluster, predictor cluster
    trainers = [S.Server(tm.address()) for _ in range(2)]
    predictors = [S.Server(pm.address())]
    syncers = []
    try:
        tc, pc = S.Client(tm.address()), S.Client(pm.address())
        psid, ph = _table(pc, {predictors[0].node_id(): [0, 1, 2]}, {})
        assert C.set_model(S.MasterClient(pm.address()), json.dumps(_model("ctr", "emb", psid, ph))).ok()
        follow = {"sync_table": [{"model_name": "ctr", "table_name": "emb", "op_key": "sync"}]}
        ids = [s.node_id() for s in trainers]
        tsid, th = _table(tc, {ids[0]: [0], ids[1]: [1]}, follow)
        syncers = [S.TableSyncer(s, pm.address(), 3, 0.05) for s in trainers]
        push = S.PushHandler(tc, tsid, th["push"])
        ppull = S.PullHandler(pc, psid, ph["pull_ro"])
        keys = np.arange(600, dtype=np.int64)
        assert push.async_push(keys, -np.ones((600, DIM), np.float32)).ok()
        assert all(s.wait_idle(10000) for s in syncers)
        st, rows = ppull.pull(keys)
        assert st.ok() and np.all(rows == 1.0)
        assert sum(s.stats()["rows"] for s in syncers) == 600 and all(s.stats()["errors"] == 0 for s in syncers)
        # only the rows that change travel afterwards
        assert push.async_push(keys[:9], -np.ones((9, DIM), np.float32)).ok()
        assert all(s.wait_idle(10000) for s in syncers)
        assert sum(s.stats()["rows"] for s in syncers) == 609
        assert np.all(ppull.pull(keys[:9])[1] == 2.0) and np.all(ppull.pull(keys[9:])[1] == 1.0)
        # buffered pushes reach the follower with the store, not before
        assert push.sync_push(keys[:5], -np.ones((5, DIM), np.float32)).ok()
        assert all(s.wait_idle(10000) for s in syncers)
        assert np.all(ppull.pull(keys[:5])[1] == 2.0)
        assert push.store().ok()
        assert _wait(lambda: np.all(ppull.pull(keys[:5])[1] == 3.0))
        # a reshard of the followed table loses nothing that is still to be shipped: push, move the shards, push
        assert push.async_push(keys[100:200], -np.ones((100, DIM), np.float32)).ok()
        assert S.UpdateContextHandler(tc, tsid, th["update_ctx"]).update_context(S.nodes_json({ids[0]: [1], ids[1]: [0]})).ok()
        assert push.async_push(keys[150:250], -np.ones((100, DIM), np.float32)).ok()
        want = S.PullHandler(tc, tsid, th["pull_ro"]).pull(keys)[1]
        assert _wait(lambda: np.array_equal(ppull.pull(keys)[1], want)), (ppull.pull(keys)[1] - want).nonzero()
        # deleting the followed table retires it from the thread's books; the predictor keeps its rows
        assert tc.delete_storage(tsid).ok()
        assert all(s.wait_idle(10000) for s in syncers)
        assert np.array_equal(ppull.pull(keys)[1], want)
    finally:
        for s in syncers:
            s.stop()
        for s in trainers + predictors:
            s.stop()
        tm.stop()
        pm.stop()


def test_a_follower_that_does_not_exist_is_an_error_not_a_hang():
    m = S.Master()
    server = S.Server(m.address())
    syncer = None
    try:
        client = S.Client(m.address())
        follow = {"sync_table": [{"model_name": "nobody", "table_name": "emb", "op_key": "sync"}]}
        sid, h = _table(client, {server.node_id(): [0]}, follow)
        syncer = S.TableSyncer(server, m.address(), 2, 0.01)
        keys = np.arange(10, dtype=np.int64)
        assert S.PushHandler(client, sid, h["push"]).async_push(keys, np.ones((10, DIM), np.float32)).ok()
        assert syncer.wait_idle(10000)
        stats = syncer.stats()
        assert stats["errors"] >= 1 and stats["rows"] == 0 and stats["last_error"]
        # the model appears later: the next push ships everything that is still marked
        fsid, fh = _table(client, {server.node_id(): [0, 1]}, {})
        assert C.set_model(S.MasterClient(m.address()), json.dumps(_model("nobody", "emb", fsid, fh))).ok()
        assert S.PushHandler(client, sid, h["push"]).async_push(keys[:1], np.ones((1, DIM), np.float32)).ok()
        assert syncer.wait_idle(10000)
        assert syncer.stats()["rows"] == 10
        st, rows = S.PullHandler(client, fsid, fh["pull_ro"]).pull(keys)
        assert st.ok() and np.all(rows[1:] == -1.0) and np.all(rows[0] == -2.0)
    finally:
        if syncer:
            syncer.stop()
        server.stop()
        m.stop()


def test_two_followers_and_one_of_them_appears_late():
    """A table with two followers: while one of them cannot be found the other still receives every change, and the
    late one gets everything once it exists (the marks stay until every follower has the rows)."""
    m = S.Master()
    server = S.Server(m.address())
    syncer = None
    try:
        client = S.Client(m.address())
        a_sid, a_h = _table(client, {server.node_id(): [0, 1]}, {})
        assert C.set_model(S.MasterClient(m.address()), json.dumps(_model("first", "emb", a_sid, a_h))).ok()
        follow = {"sync_table": [{"model_name": "late", "table_name": "emb", "op_key": "sync"},
                                 {"model_name": "first", "table_name": "emb", "op_key": "sync"}]}
        sid, h = _table(client, {server.node_id(): [0]}, follow)
        syncer = S.TableSyncer(server, m.address(), 2, 0.01)
        push = S.PushHandler(client, sid, h["push"])
        keys = np.arange(40, dtype=np.int64)
        assert push.async_push(keys, -np.ones((40, DIM), np.float32)).ok()
        assert syncer.wait_idle(10000)
        assert np.all(S.PullHandler(client, a_sid, a_h["pull_ro"]).pull(keys)[1] == 1.0)      # the follower that exists is served
        assert syncer.stats()["errors"] >= 1
        b_sid, b_h = _table(client, {server.node_id(): [0, 1, 2]}, {})
        assert C.set_model(S.MasterClient(m.address()), json.dumps(_model("late", "emb", b_sid, b_h))).ok()
        assert push.async_push(keys[:3], -np.ones((3, DIM), np.float32)).ok()
        assert syncer.wait_idle(10000)
        want = S.PullHandler(client, sid, h["pull_ro"]).pull(keys)[1]
        for fsid, fh in ((a_sid, a_h), (b_sid, b_h)):
            assert np.array_equal(S.PullHandler(client, fsid, fh["pull_ro"]).pull(keys)[1], want)
    finally:
        if syncer:
            syncer.stop()
        server.stop()
        m.stop()


def test_collective_training_table_feeds_a_predictor_table_of_the_service_layer():
    """`parallel.PredictorSync`: the rows that a collective (training) table changed travel to a predictor table of
    the RPC path in blocks; a round that the predictor refused is sent again in full, marks are cleared only after a
    whole round."""
    import torch
    from parameter_server_b200 import SparseTable
    from parameter_server_b200.parallel import PredictorSync
    from parameter_server_b200.utils.status import StatusError

    master = S.Master()
    servers = [S.Server(master.address()) for _ in range(2)]
    client = S.Client(master.address())
    try:
        ids = [s.node_id() for s in servers]
        # full rows travel: the predictor keeps the same row layout (adagrad: embedding + accumulator)
        cfg = dict(dim=DIM, optimizer="adagrad", lr=0.1, init_accumulator=0.5, init_range=0.0)
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0, 1], ids[1]: [1, 0]}, cfg))
        assert st.ok(), st
        _, h_pull = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
        _, h_sync = client.register_handler("sync", S.LIB, "KVSyncOperator", json.dumps({"block_size": 64}), sid)
        pull = S.PullHandler(client, sid, h_pull)
        train = SparseTable(DIM, "adagrad", dict(lr=0.1, init_accumulator=0.5), init_range=0.0, device="cpu", group="none")
        sync = PredictorSync(train, S.SyncHandler(client, sid, h_sync))
        assert sync.block == 64
        keys = torch.arange(1, 1001, dtype=torch.int64)
        train.pull(keys)
        train.push(-torch.ones(1000, DIM) * (keys % 5 + 1).float()[:, None])
        assert sync.sync() == 1000
        want = train.pull(keys, insert=False).numpy()
        for _ in range(4):                                                     # either replica
            st, rows = pull.pull(keys.numpy())
            assert st.ok() and np.array_equal(rows, want)
        assert sync.sync() == 0
        # only what changed travels
        some = keys[::10]
        train.pull(some)
        train.push(torch.ones(100, DIM))
        for s in servers:
            s.stop()                                                           # the predictor cluster is away
        try:
            sync.timeout_ms = 500
            sync.sync()
            raise AssertionError("a round that nobody took must raise")
        except StatusError:
            pass
        assert sync.failed_rounds == 1
        # a new predictor cluster (its table starts empty): the handler is replaced, the kept marks send the increment
        servers = [S.Server(master.address()) for _ in range(2)]
        ids = [s.node_id() for s in servers]
        st, sid2 = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0], ids[1]: [1]}, cfg))
        assert st.ok(), st
        _, h_pull2 = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid2)
        _, h_sync2 = client.register_handler("sync", S.LIB, "KVSyncOperator", "{}", sid2)
        sync.handler = S.SyncHandler(client, sid2, h_sync2)
        sync.timeout_ms = 30000
        assert sync.sync() == 100
        st, rows = S.PullHandler(client, sid2, h_pull2).pull(some.numpy())
        assert st.ok() and np.array_equal(rows, train.pull(some, insert=False).numpy())
        # embeddings only, into a predictor table without optimizer state
        st, sid3 = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                         S.storage_config({ids[0]: [0, 1, 2]}, dict(dim=DIM, optimizer="set", init_range=0.0)))
        assert st.ok(), st
        _, h_pull3 = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid3)
        _, h_sync3 = client.register_handler("sync", S.LIB, "KVSyncOperator", "{}", sid3)
        emb = PredictorSync(train, S.SyncHandler(client, sid3, h_sync3), embedding_only=True)
        assert emb.sync() == 1000
        st, rows = S.PullHandler(client, sid3, h_pull3).pull(keys.numpy())
        assert st.ok() and np.array_equal(rows, train.pull(keys, insert=False).numpy())
    finally:
        for s in servers:
            s.stop()
        master.stop()
