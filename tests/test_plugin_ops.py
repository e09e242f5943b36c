"""Operators supplied by a plug-in library: a user-written erase predicate, a user-written for_each reducer with its
own result type, a dense value partitioner and a reshard codec, registered under the plug-in's library name and run
by the servers. The reference's extension points: REGISTER_OPERATOR(lib, Class) (pico-ps/operator/Operator.h:118-130),
virtual init_result / for_each / merge_result (ForEachOperator.h:214-232), virtual erase_if (EraseIfOperator.h:57),
DenseValuePartitioner / Merger (common/dense_common.h:135-171), BaseShardUpdateContextOperator
(UpdateContextOperator.h:59-213)."""
import json
import os
import shutil
import struct
import subprocess

import numpy as np
import pytest

from parameter_server_b200 import StatusCode
from parameter_server_b200 import service as S

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "parameter_server_b200", "csrc")
DIM = 4


@pytest.fixture(scope="module")
def plugin(tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    out = str(tmp_path_factory.mktemp("plugin") / "libplugin_ops.so")
    build = subprocess.run([gxx, "-std=c++17", "-O1", "-shared", "-fPIC", "-DPSB_OPERATOR_PLUGIN", "-I", CSRC, "-I", "/usr/local/cuda/include",
                            os.path.join(HERE, "cpp", "plugin_ops.cpp"), "-o", out], capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    return out


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


def test_unknown_plugin_operator_is_refused_before_the_library_is_loaded():
    cl = Cluster(1)
    try:
        st, sid = cl.client.create_storage(S.LIB, "SparseTableStorageOperator",
                                           S.storage_config({cl.ids()[0]: [0, 1]}, dict(dim=DIM, optimizer="sum", init_range=0.0)))
        assert st.ok()
        st, _ = cl.client.register_handler("erase_plugin", "no_such_lib", "EraseEvenAbove", "{}", sid)
        assert st.code() == StatusCode.INVALID_CONFIG
    finally:
        cl.close()


def test_plugin_erase_predicate_and_reducer_run_on_the_servers(plugin):
    cl = Cluster(3)
    try:
        assert cl.client.load_operator_library(plugin).ok()       # this process and every server
        ids = cl.ids()
        nodes = {ids[0]: [0, 1], ids[1]: [2, 3, 4], ids[2]: [5]}
        st, sid = cl.client.create_storage(S.LIB, "SparseTableStorageOperator",
                                           S.storage_config(nodes, dict(dim=DIM, optimizer="sum", init_range=0.0)))
        assert st.ok(), st
        h = {}
        for key, lib, op in [("push", S.LIB, "SparseTablePushOperator"), ("pull", S.LIB, "SparseTablePullOperator"),
                             ("stats", S.LIB, "ForEachOperator"), ("hist", "testplugin", "KeyHistogram"),
                             ("erase", "testplugin", "EraseEvenAbove")]:
            st, h[key] = cl.client.register_handler(key, lib, op, json.dumps({"read_only": True} if key == "pull" else {}), sid)
            assert st.ok(), (key, st)
        keys = np.arange(10, 1010, dtype=np.int64)
        vals = np.tile((keys % 10).astype(np.float32)[:, None], (1, DIM))      # first value = key % 10
        assert S.PushHandler(cl.client, sid, h["push"]).async_push(keys, vals).ok()
        # the plug-in's reducer has its own result layout: four residue counts and the smallest key
        st, raw = S.ForEachHandler(cl.client, sid, h["hist"]).for_each_raw("{}")
        assert st.ok(), st
        b0, b1, b2, b3, kmin = struct.unpack("<5q", raw)
        assert [b0, b1, b2, b3] == [int((keys % 4 == r).sum()) for r in range(4)] and kmin == 10
        # the built-in reducer still answers through the same handler type
        st, d = S.ForEachHandler(cl.client, sid, h["stats"]).for_each("{}")
        assert st.ok() and d["count"] == 1000 and abs(d["sum"] - float(vals.sum())) < 1e-3
        # the built-in handler refuses to unpack somebody else's result bytes
        st, _ = S.ForEachHandler(cl.client, sid, h["hist"]).for_each("{}")
        assert not st.ok()
        # the plug-in's predicate: even keys whose first value exceeds the bound
        st, n = S.EraseIfHandler(cl.client, sid, h["erase"]).erase_if(json.dumps({"bound": 5.5}))
        doomed = (keys % 2 == 0) & (keys % 10 > 5.5)
        assert st.ok() and n == int(doomed.sum())
        st, d = S.ForEachHandler(cl.client, sid, h["stats"]).for_each("{}")
        assert st.ok() and d["count"] == 1000 - int(doomed.sum())
        st, rows = S.PullHandler(cl.client, sid, h["pull"]).pull(keys)
        assert st.ok()
        assert np.array_equal(rows[:, 0] != 0, ~doomed & (keys % 10 != 0))
        # the plug-in's writing scan: odd keys get their key stamped into the first value, in place on the servers
        st, hw = cl.client.register_handler("stamp", "testplugin", "StampOddKeys", "{}", sid)
        assert st.ok(), st
        st, raw = S.ForEachHandler(cl.client, sid, hw).for_each_raw("{}")
        assert st.ok() and struct.unpack("<q", raw)[0] == int((keys % 2 == 1).sum())
        st, after = S.PullHandler(cl.client, sid, h["pull"]).pull(keys)
        odd = keys % 2 == 1
        assert st.ok() and np.array_equal(after[odd, 0], keys[odd].astype(np.float32))
        assert np.array_equal(after[~odd], rows[~odd]) and np.array_equal(after[odd, 1:], rows[odd, 1:])
    finally:
        cl.close()


def test_plugin_dense_partitioner_and_reshard_codec(plugin, tmp_path):
    cl = Cluster(2)
    try:
        assert cl.client.load_operator_library(plugin).ok()
        ids = cl.ids()
        trace = str(tmp_path / "trace.txt")
        st, sid = cl.client.create_storage(S.LIB, "DenseTableStorageOperator",
                                           S.storage_config({ids[0]: [0, 1], ids[1]: [2, 3]}, dict(dim=8, optimizer="sum")))
        assert st.ok(), st
        h = {}
        for key, lib, op, cfg in [("push", "testplugin", "ReversedDensePush", {}), ("pull", "testplugin", "ReversedDensePull", {}),
                                  ("pull_plain", S.LIB, "DenseTablePullOperator", {}),
                                  ("update_ctx", "testplugin", "TracingUpdateContext", {"trace": trace})]:
            st, h[key] = cl.client.register_handler(key, lib, op, json.dumps(cfg), sid)
            assert st.ok(), (key, st)
        value = np.arange(1, 30, dtype=np.float32)                       # 29 elements: 4 slices of 8, the last one short
        assert S.PushHandler(cl.client, sid, h["push"]).push_dense(7, value).ok()
        st, back = S.PullHandler(cl.client, sid, h["pull"]).pull_dense(7, value.size)
        assert st.ok() and np.array_equal(back, value)                   # the pair agrees on the cut
        # the default cut sees the slices in the plug-in's (reversed) order: slice 0 holds the LAST block
        st, plain = S.PullHandler(cl.client, sid, h["pull_plain"]).pull_dense(7, value.size)
        assert st.ok() and np.array_equal(plain[:5], value[24:]) and np.array_equal(plain[8:16], value[16:24])
        # the table's reshard runs through the plug-in's codec
        new_nodes = {ids[0]: [0, 1, 2], ids[1]: [3, 4, 5]}
        st = S.UpdateContextHandler(cl.client, sid, h["update_ctx"]).update_context(S.nodes_json(new_nodes))
        assert st.ok(), st
        lines = open(trace).read().split("\n")
        assert sum(l.startswith("shuffle") for l in lines) == 4 and sum(l.startswith("purge") for l in lines) >= 2
        st, back = S.PullHandler(cl.client, sid, h["pull"]).pull_dense(7, value.size)
        assert st.ok() and np.array_equal(back, value)
    finally:
        cl.close()
