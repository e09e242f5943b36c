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
