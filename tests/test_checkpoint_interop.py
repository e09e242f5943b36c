"""Dump files are one format for both data paths: a dump written by the RPC servers loads into a collective-path
table and a dump written by the collective path loads into RPC servers (host back-end, one process)."""
import json

import numpy as np
import torch

from parameter_server_b200 import SparseTable
from parameter_server_b200 import service as S
from parameter_server_b200.parallel import checkpoint

DIM = 4
OPT = dict(dim=DIM, optimizer="adagrad", lr=0.1, init_accumulator=0.5, init_range=0.0)


def _rpc_table(client, ids):
    nodes = {n: [2 * i, 2 * i + 1] for i, n in enumerate(ids)}
    st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config(nodes, OPT))
    assert st.ok(), st
    h = {}
    for key, op, cfg in [("pull_ro", "SparseTablePullOperator", {"read_only": True}), ("push", "SparseTablePushOperator", {}),
                         ("dump", "DumpOperator", {}), ("load", "LoadOperator", {"block_size": 64})]:
        st, h[key] = client.register_handler(key, S.LIB, op, json.dumps(cfg), sid)
        assert st.ok(), st
    return sid, h


def test_dumps_of_the_two_paths_load_into_each_other(tmp_path):
    master = S.Master()
    servers = [S.Server(master.address()) for _ in range(2)]
    client = S.Client(master.address())
    try:
        rng = np.random.default_rng(3)
        keys = rng.choice(1 << 40, size=700, replace=False).astype(np.int64)
        grads = rng.standard_normal((700, DIM)).astype(np.float32)
        # RPC servers -> dump -> collective table
        sid, h = _rpc_table(client, [s.node_id() for s in servers])
        assert S.PushHandler(client, sid, h["push"]).async_push(keys, grads).ok()
        st, want = S.PullHandler(client, sid, h["pull_ro"]).pull(keys)
        assert st.ok()
        uri = str(tmp_path / "from_rpc") + "?format=binary"
        st, n = S.DumpHandler(client, sid, h["dump"]).dump(uri, 3)
        assert st.ok() and n == 700
        table = SparseTable(DIM, "adagrad", dict(lr=0.1, init_accumulator=0.5), n_shards=5, init_range=0.0, device="cpu", group="none")
        assert checkpoint.load(table, uri) == 700
        got = table.pull(torch.from_numpy(keys), insert=False)
        assert np.array_equal(got.numpy(), want)
        # the optimizer state travelled too: one more identical push gives identical rows on both sides
        more = rng.standard_normal((700, DIM)).astype(np.float32)
        assert S.PushHandler(client, sid, h["push"]).async_push(keys, more).ok()
        table.pull(torch.from_numpy(keys))
        table.push(torch.from_numpy(more))
        st, want2 = S.PullHandler(client, sid, h["pull_ro"]).pull(keys)
        got2 = table.pull(torch.from_numpy(keys), insert=False)
        assert np.allclose(got2.numpy(), want2, rtol=1e-6, atol=1e-7)
        # collective table -> dump -> RPC servers (a fresh table with another placement)
        uri2 = str(tmp_path / "from_collective")
        assert checkpoint.dump(table, uri2, file_number=2) == 700
        sid2, h2 = _rpc_table(client, [s.node_id() for s in servers][::-1])
        st, n = S.LoadHandler(client, sid2, h2["load"]).load(uri2 + "?format=binary")
        assert st.ok() and n == 700, st
        st, back = S.PullHandler(client, sid2, h2["pull_ro"]).pull(keys)
        assert st.ok() and np.array_equal(back, got2.numpy())
    finally:
        for s in servers:
            s.stop()
        master.stop()
