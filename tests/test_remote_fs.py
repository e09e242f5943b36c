"""Dump, load and restore through a Hadoop file system: paths with the hdfs:// scheme are served by the configured
`hadoop` command (here a stand-in that keeps the files under a local root and logs every call)."""
import json
import os
import sys

import numpy as np

from parameter_server_b200 import service as S

HERE = os.path.dirname(os.path.abspath(__file__))
DIM = 4


def test_dump_load_restore_over_the_hadoop_command(tmp_path, monkeypatch):
    root = tmp_path / "hdfs_root"
    root.mkdir()
    monkeypatch.setenv("FAKE_HDFS_ROOT", str(root))
    launcher = tmp_path / "hadoop"
    launcher.write_text(f"#!/bin/sh\nexec {sys.executable} {os.path.join(HERE, 'fake_hadoop.py')} \"$@\"\n")
    launcher.chmod(0o755)
    S.set_hadoop_bin(str(launcher))
    master = S.Master()
    servers = [S.Server(master.address()) for _ in range(2)]
    try:
        client = S.Client(master.address())
        ids = [s.node_id() for s in servers]

        def table(nodes, compress):
            st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                            S.storage_config(nodes, dict(dim=DIM, optimizer="sum", init_range=0.0)))
            assert st.ok(), st
            h = {}
            for key, op, cfg in [("push", "SparseTablePushOperator", {}), ("pull_ro", "SparseTablePullOperator", {"read_only": True}),
                                 ("dump", "DumpOperator", {"compress_algorithm": compress}),
                                 ("load", "LoadOperator", {"compress_algorithm": compress, "block_size": 100})]:
                st, h[key] = client.register_handler(key, S.LIB, op, json.dumps(cfg), sid)
                assert st.ok(), st
            return sid, h

        for compress in ("", "zstd"):
            uri = f"hdfs://namenode:8020/models/run_{compress or 'plain'}"
            sid, h = table({ids[0]: [0, 1], ids[1]: [2]}, compress)
            keys = np.arange(1200, dtype=np.int64)
            vals = ((keys[:, None] % 11 + 1) * np.ones((1, DIM))).astype(np.float32)
            assert S.PushHandler(client, sid, h["push"]).async_push(keys, vals).ok()
            st, n = S.DumpHandler(client, sid, h["dump"]).dump(uri, 2)
            assert st.ok() and n == 1200, st
            stored = sorted(os.listdir(root / "models" / f"run_{compress or 'plain'}"))
            assert len(stored) == 3 and all(f.startswith("model_") for f in stored), stored   # shards 0, 1 of one node: 2 files; shard 2: 1
            # load (rehash) into a table with another placement, straight from the remote directory
            sid2, h2 = table({ids[0]: [0], ids[1]: [1, 2, 3]}, compress)
            st, n = S.LoadHandler(client, sid2, h2["load"]).load(uri)
            assert st.ok() and n == 1200, st
            st, rows = S.PullHandler(client, sid2, h2["pull_ro"]).pull(keys)
            assert st.ok() and np.array_equal(rows, vals)
            # restore (same placement, no rehash), then drop the remote files
            sid3, h3 = table({ids[0]: [0, 1], ids[1]: [2]}, compress)
            st, n = S.LoadHandler(client, sid3, h3["load"]).restore(uri, True)
            assert st.ok(), st
            st, rows = S.PullHandler(client, sid3, h3["pull_ro"]).pull(keys)
            assert st.ok() and np.array_equal(rows, vals)
            assert os.listdir(root / "models" / f"run_{compress or 'plain'}") == []
        calls = (root / "calls.log").read_text()
        for verb in ("fs -mkdir -p hdfs://", "fs -put -f - hdfs://", "fs -ls hdfs://", "fs -cat hdfs://", "fs -rm -f hdfs://"):
            assert verb in calls, verb
        # the collective path reaches the same directory: an RPC-server dump loads into a collective table and back
        import torch
        from parameter_server_b200 import SparseTable
        from parameter_server_b200.parallel import checkpoint
        sid4, h4 = table({ids[0]: [0, 1], ids[1]: [2]}, "")
        assert S.PushHandler(client, sid4, h4["push"]).async_push(keys, vals).ok()
        assert S.DumpHandler(client, sid4, h4["dump"]).dump("hdfs://namenode:8020/models/shared", 2)[0].ok()
        t = SparseTable(DIM, "sum", n_shards=3, init_range=0.0, device="cpu", group="none")
        assert checkpoint.load(t, "hdfs://namenode:8020/models/shared") == 1200
        assert np.array_equal(t.pull(torch.from_numpy(keys), insert=False).numpy(), vals)
        assert checkpoint.dump(t, "hdfs://namenode:8020/models/from_collective", file_number=2) == 1200
        sid5, h5 = table({ids[0]: [0], ids[1]: [1]}, "")
        st, n = S.LoadHandler(client, sid5, h5["load"]).load("hdfs://namenode:8020/models/from_collective")
        assert st.ok() and n == 1200, st
        assert np.array_equal(S.PullHandler(client, sid5, h5["pull_ro"]).pull(keys)[1], vals)
        # a command that is not there is an error for the caller, not a crash
        S.set_hadoop_bin(str(tmp_path / "no_such_hadoop"))
        st, _ = S.DumpHandler(client, sid, h["dump"]).dump("hdfs://namenode:8020/models/other", 1, 5000)
        assert not st.ok()
    finally:
        S.set_hadoop_bin("")
        for s in servers:
            s.stop()
        master.stop()
