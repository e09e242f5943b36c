#!/usr/bin/env python
"""Config 1 of the benchmark: the CPU restatement of the reference algorithm, timed.

2 pserver processes + 2 worker processes on localhost (plus a master), one sparse table: int64 keys
drawn Zipf(1.1) from 1 M distinct keys in [0, 2^40), dim 16 fp32, uniform(-0.01, 0.01) init, Adagrad(lr 0.05,
initial accumulator 0.1). Every step a worker pulls 8192 keys and pushes N(0, 1e-3) gradients for the same
keys; seed 0; `--steps` steps per worker (1000 in the config); then dump -> load into a fresh table -> bitwise
comparison. The servers run the C++ host storage (client dedup map -> jump-consistent-hash partition ->
per-shard locked hash map, the reference's structure) behind the TCP service layer.

    python baseline/cpu_restatement.py [--steps 1000] [--gpu]     # --gpu: the same loop on one B200 (fused kernels)

Prints one JSON line: keys/s for pull, push and pull+push (wall clock over all workers).
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

DIM, BATCH, DISTINCT = 16, 8192, 1_000_000
OP_CFG = dict(dim=DIM, optimizer="adagrad", lr=0.05, init_accumulator=0.1, init_range=0.01, seed=0)


def key_pool(seed=0):
    rng = np.random.default_rng(seed)
    return np.unique(rng.integers(0, 1 << 40, size=int(DISTINCT * 1.05)))[:DISTINCT]


def batches(rank, steps, pool):
    rng = np.random.default_rng(100 + rank)
    for _ in range(steps):
        ranks = (rng.zipf(1.1, size=BATCH) - 1) % DISTINCT
        yield pool[ranks], (rng.standard_normal((BATCH, DIM)) * 1e-3).astype(np.float32)


def pserver(master_addr, ready, stop):
    from parameter_server_b200 import service as S
    server = S.Server(master_addr)
    ready.put(server.node_id())
    stop.wait()
    server.stop()


def worker(rank, master_addr, sid, hids, steps, out):
    from parameter_server_b200 import service as S
    client = S.Client(master_addr)
    assert client.initialize_storage(sid).ok()
    pull, push = S.PullHandler(client, sid, hids["pull"]), S.PushHandler(client, sid, hids["push"])
    pool = key_pool()
    t_pull = t_push = 0.0
    for keys, grads in batches(rank, steps, pool):
        t0 = time.perf_counter()
        st, _ = pull.pull(keys)
        t1 = time.perf_counter()
        assert st.ok(), st
        st = push.async_push(keys, grads)
        t2 = time.perf_counter()
        assert st.ok(), st
        t_pull += t1 - t0
        t_push += t2 - t1
    out.put((rank, t_pull, t_push))


def run_cpu(steps):
    from parameter_server_b200 import service as S
    mp.set_start_method("spawn", force=True)
    master = S.Master()
    ready, stop = mp.Queue(), mp.Event()
    servers = [mp.Process(target=pserver, args=(master.address(), ready, stop)) for _ in range(2)]
    [p.start() for p in servers]
    ids = sorted(ready.get() for _ in servers)
    client = S.Client(master.address())
    st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0, 1], ids[1]: [2, 3]}, OP_CFG))
    assert st.ok(), st
    hids = {}
    for key, op in [("pull", "SparseTablePullOperator"), ("push", "SparseTablePushOperator"), ("dump", "DumpOperator"),
                    ("load", "LoadOperator")]:
        st, hids[key] = client.register_handler(key, S.LIB, op, "{}", sid)
        assert st.ok(), st
    out = mp.Queue()
    workers = [mp.Process(target=worker, args=(r, master.address(), sid, hids, steps, out)) for r in range(2)]
    t0 = time.perf_counter()
    [p.start() for p in workers]
    res = [out.get() for _ in workers]
    [p.join() for p in workers]
    wall = time.perf_counter() - t0
    # dump -> load -> bitwise
    tmp = tempfile.mkdtemp(prefix="psb_cfg1_")
    st, n = S.DumpHandler(client, sid, hids["dump"]).dump(tmp + "/dump", 2)
    assert st.ok(), st
    st, sid2 = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0], ids[1]: [1, 2]}, OP_CFG))
    h2 = {}
    for key, op in [("pull", "SparseTablePullOperator"), ("load", "LoadOperator")]:
        st, h2[key] = client.register_handler(key, S.LIB, op, json.dumps({"read_only": True}), sid2)
    st, n2 = S.LoadHandler(client, sid2, h2["load"]).load(tmp + "/dump")
    assert st.ok() and n2 == n, (st, n, n2)
    probe = key_pool()[:50000]
    st, rp = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
    a = S.PullHandler(client, sid, rp).pull(probe)[1]
    b = S.PullHandler(client, sid2, h2["pull"]).pull(probe)[1]
    bitwise = a.tobytes() == b.tobytes()
    stop.set()
    [p.join(10) for p in servers]
    master.stop()
    total = 2 * steps * BATCH
    tp = max(r[1] for r in res)
    tq = max(r[2] for r in res)
    return {"impl": "cpu_restatement", "servers": 2, "workers": 2, "steps_per_worker": steps, "keys_per_step": BATCH,
            "pull_keys_per_sec": total / tp, "push_keys_per_sec": total / tq, "pull_push_keys_per_sec": 2 * total / (tp + tq),
            "wall_s": wall, "table_rows": int(n), "dump_load_bitwise_equal": bool(bitwise)}


def run_gpu(steps):
    import torch
    from parameter_server_b200 import SparseTable
    t = SparseTable(DIM, "adagrad", dict(lr=0.05, init_accumulator=0.1), capacity=2 * DISTINCT, max_keys=BATCH, seed=0)
    pool = key_pool()
    data = [(torch.from_numpy(k).pin_memory(), torch.from_numpy(g).pin_memory()) for k, g in batches(0, min(steps, 64), pool)]
    dk = torch.empty(BATCH, dtype=torch.int64, device="cuda")
    dg = torch.empty((BATCH, DIM), device="cuda")
    out = torch.empty((BATCH, DIM), device="cuda")
    t.reserve(DISTINCT)
    for i in range(8):
        dk.copy_(data[i % len(data)][0]); t.pull(dk, out=out); dg.copy_(data[i % len(data)][1]); t.push(dg)
    t.check()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(steps):
        k, g = data[i % len(data)]
        dk.copy_(k, non_blocking=True); dg.copy_(g, non_blocking=True)
        t.pull(dk, out=out)
        t.push(dg)
    e1.record()
    torch.cuda.synchronize()
    t.check()
    sec = e0.elapsed_time(e1) * 1e-3
    return {"impl": "ours_1gpu_fused", "steps": steps, "keys_per_step": BATCH, "pull_push_keys_per_sec": 2 * steps * BATCH / sec,
            "us_per_step": sec / steps * 1e6, "includes": "H2D copy of keys and gradients from pinned memory every step",
            "table_rows": t.size()}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--gpu", action="store_true")
    a = ap.parse_args()
    print(json.dumps(run_gpu(a.steps) if a.gpu else run_cpu(a.steps)))
