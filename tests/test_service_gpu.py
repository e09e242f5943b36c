"""The RPC service path with the GPU storage back-end: servers keep their shards in HBM and serve
host requests through the fused kernels."""
import json

import numpy as np
import pytest

from parameter_server_b200 import service as S
from test_service import Cluster, make_table, uneven

pytestmark = pytest.mark.gpu


def test_gpu_backed_servers_end_to_end(tmp_path):
    cl = Cluster(2)
    try:
        cfg = dict(dim=16, optimizer="adagrad", lr=0.05, init_accumulator=0.1, init_range=0.01, backend="gpu", device=0,
                   capacity=1 << 16, max_batch=1 << 14)
        host_cfg = dict(cfg, backend="host")
        sid, h = make_table(cl, uneven(cl.ids()), cfg=cfg)
        ref, hr = make_table(cl, uneven(cl.ids()), cfg=host_cfg)
        rng = np.random.default_rng(0)
        keys = rng.integers(0, 1 << 40, size=20000)
        grads = rng.standard_normal((20000, 16)).astype(np.float32) * 1e-2
        for s_, hh in ((sid, h), (ref, hr)):
            pull, push = S.PullHandler(cl.client, s_, hh["pull"]), S.PushHandler(cl.client, s_, hh["push"])
            assert pull.pull(keys)[0].ok()
            assert push.async_push(keys, grads).ok()
        a = S.PullHandler(cl.client, sid, h["pull_ro"]).pull(keys)[1]
        b = S.PullHandler(cl.client, ref, hr["pull_ro"]).pull(keys)[1]
        assert a.tobytes() == b.tobytes()          # same init, same update rule, bit for bit
        # dump from HBM, load into the host table of another sharding, compare
        uri = str(tmp_path / "gpu_dump")
        st, n = S.DumpHandler(cl.client, sid, h["dump"]).dump(uri, 2)
        assert st.ok() and n == len(set(keys.tolist()))
        sid2, h2 = make_table(cl, {cl.ids()[0]: [0, 1, 2]}, cfg=cfg)
        assert S.LoadHandler(cl.client, sid2, h2["load"]).load(uri)[0].ok()
        c = S.PullHandler(cl.client, sid2, h2["pull_ro"]).pull(keys)[1]
        assert c.tobytes() == a.tobytes()
        st, erased = S.EraseIfHandler(cl.client, sid2, h2["erase_if"]).erase_if(json.dumps({"type": "key_mod", "mod": 2, "rem": 0}))
        assert st.ok() and erased == sum(1 for k in set(keys.tolist()) if k % 2 == 0)
        # reshard a GPU table
        new = {cl.ids()[0]: [0, 1], cl.ids()[1]: [2, 3]}
        assert S.UpdateContextHandler(cl.client, sid, h["update_ctx"]).update_context(S.nodes_json(new)).ok()
        assert S.PullHandler(cl.client, sid, h["pull_ro"]).pull(keys)[1].tobytes() == a.tobytes()
    finally:
        cl.close()


def test_scans_run_on_the_device_and_agree_with_the_host_table():
    """erase_if with every built-in predicate and the for_each statistics of every row section: the GPU back-end
    evaluates them in one kernel over its slot array (pico-ps/operator/EraseIfOperator.h:39-48 and
    ForEachOperator.h:182-191 iterate the shard in place), the host back-end scans exported rows; both must agree."""
    cl = Cluster(2)
    try:
        cfg = dict(dim=16, optimizer="adagrad", lr=0.05, init_accumulator=0.1, init_range=0.01, backend="gpu", device=0,
                   capacity=1 << 16, max_batch=1 << 14)
        tabs = [make_table(cl, uneven(cl.ids()), cfg=c) for c in (cfg, dict(cfg, backend="host"))]
        rng = np.random.default_rng(3)
        keys = rng.integers(-(1 << 40), 1 << 40, size=12000)
        grads = (rng.standard_normal((12000, 16)) * (1 + keys[:, None] % 5)).astype(np.float32) * 1e-1
        for sid, h in tabs:
            assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, grads).ok()
        n_live = len(set(keys.tolist()))

        def stats(section):
            out = []
            for sid, h in tabs:
                st, d = S.ForEachHandler(cl.client, sid, h["for_each"]).for_each(json.dumps({"section": section}))
                assert st.ok(), st
                out.append(d)
            return out

        for section in (0, 1):
            g, hst = stats(section)
            assert g["count"] == hst["count"] == n_live
            assert abs(g["sum"] - hst["sum"]) <= 1e-6 * max(1.0, abs(hst["sum"])) + 1e-3
            assert abs(g["sum_sq"] - hst["sum_sq"]) <= 1e-6 * hst["sum_sq"] + 1e-6
            assert g["max_abs"] == hst["max_abs"]
        assert not S.ForEachHandler(cl.client, tabs[0][0], tabs[0][1]["for_each"]).for_each(json.dumps({"section": 5}))[0].ok()
        for pred in ({"type": "key_mod", "mod": 3, "rem": 1}, {"type": "l2_below", "threshold": 0.6},
                     {"type": "slot0_below", "threshold": 0.12}, {"type": "all"}):
            erased = []
            for sid, h in tabs:
                st, n = S.EraseIfHandler(cl.client, sid, h["erase_if"]).erase_if(json.dumps(pred))
                assert st.ok(), (pred, st)
                erased.append(n)
            assert erased[0] == erased[1], (pred, erased)
            g, hst = stats(0)
            assert g["count"] == hst["count"] and abs(g["sum"] - hst["sum"]) <= 1e-6 * max(1.0, abs(hst["sum"])) + 1e-3
        assert stats(0)[0]["count"] == 0
        st, _ = S.EraseIfHandler(cl.client, tabs[0][0], tabs[0][1]["erase_if"]).erase_if(json.dumps({"type": "nonsense"}))
        assert not st.ok()
    finally:
        cl.close()


def test_gpu_table_refuses_reserved_keys_from_the_network():
    """INT64_MIN and INT64_MIN + 1 mark empty and erased slots of the GPU index: a request that carries one is
    answered with an error before anything is launched, and the table keeps serving."""
    cl = Cluster(1)
    try:
        cfg = dict(dim=8, optimizer="sum", init_range=0.0, backend="gpu", device=0, capacity=1 << 12, max_batch=1 << 10)
        sid, h = make_table(cl, {cl.ids()[0]: [0, 1]}, cfg=cfg)
        pull, push = S.PullHandler(cl.client, sid, h["pull"]), S.PushHandler(cl.client, sid, h["push"])
        good = np.arange(100, dtype=np.int64)
        assert push.async_push(good, np.ones((100, 8), np.float32)).ok()
        for reserved in (-(1 << 63), -(1 << 63) + 1):
            bad = good.copy()
            bad[3] = reserved
            assert not pull.pull(bad)[0].ok()
            assert not push.async_push(bad, np.ones((100, 8), np.float32)).ok()
        st, rows = pull.pull(good)
        assert st.ok() and np.array_equal(rows, np.ones((100, 8), np.float32))
    finally:
        cl.close()


def test_gpu_push_is_all_or_nothing_when_the_row_pool_runs_out():
    """A push that cannot get a row for every key reports OUT_OF_MEMORY before it applies anything, so the client's
    retry after the table has room applies every gradient exactly once (pico-ps/handler/Handler.cpp:65-103)."""
    cl = Cluster(1)
    try:
        # an index of 8192 slots that may not grow (max_rows fixes the table's size): the fifth batch of 2048 new keys
        # finds no slot any more
        cfg = dict(dim=16, optimizer="sum", init_range=0.0, backend="gpu", device=0, capacity=1 << 12, max_batch=1 << 12,
                   max_rows=8192)
        sid, h = make_table(cl, {cl.ids()[0]: [0]}, cfg=cfg)
        pull_ro, push = S.PullHandler(cl.client, sid, h["pull_ro"]), S.PushHandler(cl.client, sid, h["push"])
        applied = []
        failed_batch = None
        for step in range(8):
            keys = np.arange(step * 2048, (step + 1) * 2048, dtype=np.int64) * 7919
            g = np.full((2048, 16), float(step + 1), np.float32)
            st = push.async_push(keys, g, 300)          # short time-out: no waiting for a reshard that never comes
            if st.ok():
                applied.append((keys, g))
            else:
                failed_batch = (keys, g)
                break
        assert failed_batch is not None and len(applied) >= 3, "the index never filled up"
        # nothing of the refused batch was applied
        st, rows = pull_ro.pull(failed_batch[0])
        assert st.ok() and not rows.any()
        # every accepted batch was applied exactly once, also after the refused one
        for keys, g in applied:
            st, rows = pull_ro.pull(keys)
            assert st.ok() and np.array_equal(rows, g)
        # room returns (keys are erased): the retry of the refused batch is applied exactly once
        st, n = S.EraseIfHandler(cl.client, sid, h["erase_if"]).erase_if(json.dumps({"type": "key_mod", "mod": 2, "rem": 0}))
        assert st.ok() and n > 0
    finally:
        cl.close()
