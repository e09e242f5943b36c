"""Elastic rescaling + HA benchmark of the collective path (benchmark config 5).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29533 \\
        -m parameter_server_b200.utils.elastic_bench --keys 134217728

A table of ``--keys`` int64 keys (dim 32 fp32 + FTRL z / n slots) is first served by half of the ranks.
Under a pull + push load of Zipf(1.1) batches (``--batch`` keys per GPU per step) it is rebalanced onto
all ranks in ``--stages`` steps of shard migration over NVLink peer copies, with load steps between the
stages (one-time start-up costs of the joining ranks are paid in a warm-up and reported separately). Then every rank's shards are mirrored on a neighbour (2x replication, full + incremental sync),
one rank loses its table (its contents are cleared on the host side, as if its process had been
replaced) and is restored from the mirror, and once more from a dump. Every time is taken with CUDA
events around the operation on each rank, maximum over ranks; rank 0 prints one JSON line.

The reference does the same through UpdateContextHandler / RestoreOperator / LoadOperator on CPU servers
(pico-ps/handler/UpdateContextHandler.cpp:62-153, pico-ps/operator/RestoreOperator.h:94-151).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import tempfile

import numpy as np
import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--keys", type=int, default=1 << 27)
    ap.add_argument("--batch", type=int, default=1 << 19)
    ap.add_argument("--stages", type=int, default=4)
    ap.add_argument("--steps", type=int, default=10, help="load steps per measurement window")
    ap.add_argument("--lost-rank", type=int, default=1)
    ap.add_argument("--dump-dir", default="")
    ap.add_argument("--reads-during", action="store_true", help="issue one read-only pull between the rounds of every migration stage")
    ap.add_argument("--no-dump", action="store_true", help="skip the dump / restore-from-dump part (it writes the whole table to disk)")
    a = ap.parse_args()

    from parameter_server_b200 import SparseTable
    from parameter_server_b200.utils.keys import zipf_batch
    from parameter_server_b200.parallel import PeerInbox, ReplicaSet, checkpoint, reshard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank = dist.get_rank() if world > 1 else 0
    dev = torch.device("cuda", local)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def rank_max(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def rank_sum(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def timed(fn):
        """fn() bracketed by barrier + CUDA events; milliseconds, max over ranks. Returns (ms, result)."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = fn()
        e1.record()
        torch.cuda.synchronize()
        return rank_max(e0.elapsed_time(e1)), r

    K, B = a.keys, a.batch
    serving0 = max(1, world // 2)
    n_shards = 8 * world
    owner0 = [s % serving0 for s in range(n_shards)]
    owner1 = [s % world for s in range(n_shards)]
    t = SparseTable(32, "ftrl", dict(lr=0.05), n_shards=n_shards, capacity=int(K / serving0 * 1.15) + (1 << 16),
                    max_keys=B, wait_limit_s=20.0, pair_capacity=min(B, B // serving0 + B // 16 + 4096))
    t.set_shard_owner(owner0)
    stride_bytes = t.table.stride() * 4 + 8

    # ---- populate: rank r inserts the keys r, r + world, ... --------------------------------------
    out = torch.empty(B, 32, device=dev)
    if rank < serving0:
        t.reserve(int(K / serving0 * 1.02) + 4 * B, exact=True)

    def populate():
        per = (K + world - 1) // world
        for lo in range(0, per, B):
            n = min(B, per - lo)
            ks = (torch.arange(lo, lo + n, device=dev, dtype=torch.int64) * world + rank).clamp_(max=K - 1)
            if n < B:
                ks = torch.cat([ks, ks[-1:].expand(B - n)])
            t.pull(ks, out=out, for_push=False)
    pop_ms, _ = timed(populate)
    t.check()
    rows_total = int(rank_sum(t.size()))

    # ---- load generator ---------------------------------------------------------------------------
    rng = np.random.default_rng(100 + rank)
    pool = []
    for _ in range(4):
        pool.append(torch.from_numpy(zipf_batch(rng, B, 1.1, K)).to(dev))
    grads = torch.randn(B, 32, device=dev) * 1e-3
    it = [0]

    def load_steps(n):
        for _ in range(n):
            t.pull(pool[it[0] % 4], out=out)
            t.push(grads)
            it[0] += 1

    def throughput(n):
        ms, _ = timed(lambda: load_steps(n))
        t.check()
        return 2.0 * B * world * n / (ms / 1e3)

    load_steps(3)
    res = {"metric": "elastic_rescale_and_restore", "n_gpus": world, "keys": K, "rows_in_table": rows_total, "dim": 32,
           "optimizer": "ftrl", "batch_per_gpu": B, "n_shards": n_shards, "populate_ms": pop_ms,
           "keys_per_sec_before": throughput(a.steps)}

    # ---- rebalance serving0 -> world ranks in stages, load running between the stages ---------------
    inbox = PeerInbox(t, 1 << 20)
    # One-time costs of a rank that has just joined (NCCL point-to-point connections for the count exchange,
    # lazy kernel loading, the stream-ordered allocator's pool, first touch of every peer's inbox) are paid
    # here, by moving one scratch row between every pair of ranks, and reported on their own.
    def warm():
        from parameter_server_b200.parallel.migrate import exchange_by_keys
        scratch = SparseTable(32, "ftrl", dict(lr=0.05), capacity=4096, max_keys=1024, group="none")
        ks = torch.arange(world, device=dev, dtype=torch.int64) + (1 << 50)
        scratch.set_rows(ks, torch.zeros(world, scratch.table.stride(), device=dev))
        exchange_by_keys(scratch, ks, [1] * world, inbox, scratch, t)
        scratch.erase_keys(ks)
        reshard(t, owner0, batch=1 << 20, inbox=inbox)      # nothing moves
        # the allocator's pool for the largest temporaries of a stage (destination sort of the keys that leave): the
        # first sort of that size otherwise pays ~100 ms of cudaMalloc inside the first stage
        n_tmp = max(1, t.size() // max(1, a.stages) + 1)
        d = torch.zeros(n_tmp, dtype=torch.int64, device=dev)
        o = torch.argsort(d, stable=True)
        _ = d[o], torch.bincount(d, minlength=world)
        del d, o, _
        torch.cuda.synchronize()
    ms, _ = timed(warm)
    res["one_time_warmup_ms"] = ms
    # the joining ranks allocate their row pools first (the create-storage step of a scale-out), timed on its own
    ms, _ = timed(lambda: t.reserve(int(K / world * 1.1) + 4 * B, exact=True) if rank >= serving0 else None)
    res["joining_ranks_alloc_ms"] = ms
    moving = [s for s in range(n_shards) if owner0[s] != owner1[s]]
    cur = list(owner0)
    reads_done = [0]

    def read_between():     # one read-only pull per exchange round: reads are served while rows move
        t.pull(pool[it[0] % 4], out=out, insert=False, for_push=False)
        it[0] += 1
        reads_done[0] += 1

    stage_ms, during, phases = [], [], []
    moved_rows = 0
    per_stage = (len(moving) + a.stages - 1) // a.stages
    for j in range(a.stages):
        # consecutive moving shards: every stage involves every (old owner -> new owner) pair, so all NVLink pairs
        # carry rows at the same time (a strided choice would single out one pair per stage)
        for s in moving[j * per_stage:(j + 1) * per_stage]:
            cur[s] = owner1[s]
        st = {}
        ms, got = timed(lambda: reshard(t, cur, batch=1 << 20, inbox=inbox, stats=st,
                                        between_rounds=read_between if a.reads_during else None))
        phases.append({k: round(v, 2) for k, v in st.items()})
        moved_rows += int(rank_sum(got))
        stage_ms.append(ms)
        during.append(throughput(max(2, a.steps // 2)))
    res.update({"rebalance_ms_total": sum(stage_ms), "rebalance_stage_ms": stage_ms, "read_only_pulls_during_rebalance": reads_done[0],
                "read_keys_per_sec_during_rebalance": reads_done[0] * B * world / (sum(stage_ms) / 1e3), "rebalance_stage_phases_rank0_ms": phases, "rows_moved": moved_rows,
                "rebalance_gbytes": moved_rows * stride_bytes / 1e9,
                "rebalance_gbytes_per_sec": moved_rows * stride_bytes / 1e9 / (sum(stage_ms) / 1e3),
                "keys_per_sec_between_stages": during, "keys_per_sec_after": throughput(a.steps),
                "rows_after": int(rank_sum(t.size()))})

    # ---- 2x replication: full mirror, then incremental -------------------------------------------
    rs = ReplicaSet(t, batch=1 << 20)
    ms, sent = timed(rs.sync)
    res.update({"replica_full_sync_ms": ms, "replica_full_sync_rows": int(rank_sum(sent))})
    load_steps(2)
    ms, sent = timed(rs.sync)
    res.update({"replica_incremental_sync_ms": ms, "replica_incremental_rows": int(rank_sum(sent))})

    # ---- one rank loses its table; restore from the mirror -----------------------------------------
    lost = a.lost_rank % world
    probe = pool[0][:4096]
    want = t.pull(probe, out=out[:4096].clone(), insert=False, for_push=False).clone()
    size_lost = t.size()
    dump_dir = [a.dump_dir or (tempfile.mkdtemp(prefix="psb_elastic_") if rank == 0 else None)]
    if world > 1:
        dist.broadcast_object_list(dump_dir, src=0)
    if rank == lost:
        t.clear()
    ms, got = timed(lambda: rs.restore(lost))
    ok = bool(torch.equal(t.pull(probe, out=out[:4096].clone(), insert=False, for_push=False), want)) and t.size() == size_lost
    res.update({"restore_from_replica_ms": ms, "restore_rows": int(rank_sum(got)), "restore_from_replica_exact": bool(rank_sum(0.0 if ok else 1.0) == 0),
                "keys_per_sec_after_restore": throughput(a.steps)})

    # ---- and from a dump (only the lost rank's files are read, the ranks share the work) ---------------
    if not a.no_dump:
        want = t.pull(probe, out=out[:4096].clone(), insert=False, for_push=False).clone()
        ms, _ = timed(lambda: checkpoint.dump(t, dump_dir[0], file_number=2))
        res["dump_ms"] = ms
        size_lost = t.size()
        if rank == lost:
            t.clear()
        ms, got = timed(lambda: checkpoint.load(t, dump_dir[0], batch=1 << 20, inbox=inbox, only_node=lost))
        ok = bool(torch.equal(t.pull(probe, out=out[:4096].clone(), insert=False, for_push=False), want)) and t.size() == size_lost
        res.update({"restore_from_dump_ms": ms, "restore_from_dump_exact": bool(rank_sum(0.0 if ok else 1.0) == 0)})
    t.check()
    barrier()
    if rank == 0:
        if not a.dump_dir:
            shutil.rmtree(dump_dir[0], ignore_errors=True)
        print(json.dumps(res))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
