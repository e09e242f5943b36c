"""Sparse key-value micro-benchmark over 1..8 GPUs (benchmark config 2).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29534 \\
        -m parameter_server_b200.utils.sparse_bench --rows-per-gpu 62500000 --impl ours

One table of ``world * rows-per-gpu`` int64 keys (62.5 M per GPU = 500 M keys on 8 GPUs), dim 64 fp32 +
an Adagrad slot, sharded by key hash and populated before anything is timed. Pull and pull+push key
throughput over batch sizes 64 Ki .. 4 Mi keys per GPU per step; keys Zipf(1.05) over the whole table
at least 30 % of the positions of a batch repeat another key of the batch (Zipf alone already gives more). CUDA events
on the launching stream, maximum over ranks; the batches rotate through four different key sets and the
rows touched per step exceed L2 from 256 Ki keys up. ``--impl nccl`` runs the NCCL-only baseline
(torch.unique + all_to_all_single) on the same table code. Rank 0 prints one JSON line per batch size.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist


def sweep(sizes, rows_per_gpu: int, impl: str = "ours", dim: int = 64, steps: int = 10, warmup: int = 3,
          phases: bool = False, emit=None):
    """Runs the sweep on the already initialised process group (or a single GPU) and returns one dict per batch
    size; ``emit`` (rank 0 only) is called with each dict as soon as it is measured."""
    from parameter_server_b200 import SparseTable
    from parameter_server_b200.parallel import NcclSparseTable
    from parameter_server_b200.utils.keys import zipf_batch

    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank() if world > 1 else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    nmax = max(sizes)
    K = rows_per_gpu * world

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

    cls = SparseTable if impl == "ours" else NcclSparseTable
    t = cls(dim, "adagrad", dict(lr=0.05, init_accumulator=0.1), capacity=int(rows_per_gpu * 1.1) + nmax, max_keys=nmax, seed=3)
    t.reserve(int(rows_per_gpu * 1.05) + 2 * nmax, exact=True)
    out = torch.empty(nmax, dim, device=dev)
    grads = torch.randn(nmax, dim, device=dev) * 1e-3
    # populate: rank r inserts keys r, r + world, ...
    for lo in range(0, rows_per_gpu, nmax):
        n = min(nmax, rows_per_gpu - lo)
        ks = torch.arange(lo, lo + n, device=dev, dtype=torch.int64) * world + rank
        t.pull(ks, out=out[:n], for_push=False)
    t.check()
    barrier()
    rows = int(rank_max(t.size()))

    rng = np.random.default_rng(77 + rank)
    results = []
    for n in sizes:
        pool = []
        for _ in range(4):
            k = zipf_batch(rng, n, 1.05, K, 0.3)
            pool.append(torch.from_numpy(k).to(dev))
        uniq = float(np.mean([torch.unique(p).numel() / n for p in pool]))
        o, g = out[:n], grads[:n]
        for i in range(warmup):
            t.pull(pool[i % 4], out=o)
            t.push(g)
        t.check()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(steps):
            t.pull(pool[i % 4], out=o, for_push=False)
        e1.record()
        torch.cuda.synchronize()
        pull_ms = rank_max(e0.elapsed_time(e1)) / steps
        barrier()
        e0.record()
        for i in range(steps):
            t.pull(pool[i % 4], out=o)
            t.push(g)
        e1.record()
        torch.cuda.synchronize()
        both_ms = rank_max(e0.elapsed_time(e1)) / steps
        t.check()
        ph = None
        if phases and impl == "ours":
            t.engine.set_profile(True)
            barrier()
            t.pull(pool[0], out=o)
            t.push(g)
            torch.cuda.synchronize()
            st = t.engine.phase_stamps(0)
            t.engine.set_profile(False)
            names = ["P1_dedup", "P2_ship_keys", "P3a_resolve", "P3b_init", "P3c_rows", "P5_gather"]
            ph = {nm: round((st[i + 1] - st[i]) / 1e3, 1) for i, nm in enumerate(names)}
            if world > 1:
                ph.update({"Q01_chain_segsum_ack_wait": round((st[9] - st[8]) / 1e3, 1), "Q2_ship_wait_grads": round((st[10] - st[9]) / 1e3, 1)})
            else:
                ph["Q1_segsum"] = round((st[10] - st[8]) / 1e3, 1)
            ph["Q3_fold_update"] = round((st[12] - st[11]) / 1e3, 1)
        # bytes that one pull + push must move through this GPU's HBM at least once: keys in, rows out, gradients in,
        # and for every distinct key its row + optimizer slot read and written
        row_b = dim * 4
        algo_bytes = n * 8 + n * row_b + n * row_b + uniq * n * (2 * 2 * row_b)
        res = {"metric": "sparse_pull_push_keys_per_sec", "phases_us_rank0": ph, "impl": impl, "n_gpus": world,
               "keys_per_gpu_per_step": n, "table_rows_max_per_gpu": rows, "table_keys": K, "dim": dim, "optimizer": "adagrad",
               "zipf_s": 1.05, "unique_fraction": uniq, "pull_ms": pull_ms, "pull_push_ms": both_ms,
               "pull_keys_per_sec": n * world / (pull_ms / 1e3),
               # every key goes through a pull AND a push in one step: counted once here ...
               "pull_push_steps_keys_per_sec": n * world / (both_ms / 1e3),
               # ... and twice (one pull + one push = two key operations) here
               "pull_push_keys_per_sec": 2 * n * world / (both_ms / 1e3),
               "pull_push_algorithmic_gbs_per_gpu": algo_bytes / (both_ms / 1e3) / 1e9}
        results.append(res)
        if emit is not None and rank == 0:
            emit(res)
    del t
    torch.cuda.empty_cache()
    return results


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows-per-gpu", type=int, default=1 << 24)
    ap.add_argument("--sizes", default="65536,262144,1048576,4194304")
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl"])
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--phases", action="store_true", help="add rank 0's in-kernel phase times of one pull + push (fused path only)")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sweep([int(s) for s in a.sizes.split(",")], a.rows_per_gpu, a.impl, a.dim, a.steps, a.warmup, a.phases,
          emit=lambda r: print(json.dumps(r), flush=True))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
