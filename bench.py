#!/usr/bin/env python
"""Headline benchmark: DLRM-style CTR training against the parameter server (samples/s, whole job),
plus the sparse pull+push key throughput of the same tables.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 the script is started once per GPU by ``python -m torch.distributed.run`` (it re-executes
itself that way when started plainly). Prints ONE JSON line on rank 0.

What is timed (own arm):
  value  device time (CUDA events, max over ranks) of K training steps, each including the
         host->device copy of that step's batch from pinned memory, the fused sparse pull, the
         tcgen05 MLP forward/backward, the fused sparse push and the fused dense push;
  e2e    the same K steps through the public call ``DLRM.train_step`` + ``read_loss`` with the loss
         read back to the host (device->host) and a stream synchronisation EVERY step.
Weak scaling: batch per GPU is fixed (global batch 65536 at 8 GPUs). Data is synthetic (per-field
Zipf keys, log-normal dense features, Bernoulli labels), weights are random-init, keys are new to the
table the first time they appear (pull inserts), so the table grows during the run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REF_UNAVAILABLE = ("reference is a C++/CMake project with no Python packaging: `pip install` reports \"Neither "
                   "'setup.py' nor 'pyproject.toml' found\", and its prpc dependency (pico-core git submodule) is "
                   "not checked out, so it cannot be built offline")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl_baseline"],
                    help="ours: fused kernels; nccl_baseline: the same model with NCCL-only sparse / dense paths (our own baseline)")
    ap.add_argument("--batch-per-gpu", type=int, default=8192)
    ap.add_argument("--no-sparse-micro", action="store_true", help="skip the sparse pull+push microbenchmark")
    ap.add_argument("--breakdown", action="store_true", help="after the timed regions, add per-section device times of an eager step")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a CUDA graph")
    ap.add_argument("--micro-keys", type=int, default=1 << 20, help="keys per GPU per step of the microbenchmark")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of this process's GPU with nvidia-smi during a region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str):
        self.uuid = uuid
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self) -> None:
        """Samples taken before this call (warm-up) are ignored by stop()."""
        self.first = len(self.lines)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        region = self.lines[getattr(self, "first", 0):] or self.lines
        for ln in region:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 8:
                continue
            try:
                sm.append(float(p[0]))
                smax.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reexec_under_torchrun(args) -> None:
    port = 29500 + (os.getpid() % 2000)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
    raise SystemExit(subprocess.call(cmd))


def main():
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:   # one line, also when launched once per GPU
            print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        reexec_under_torchrun(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import parameter_server_b200 as ps  # noqa: F401
    from parameter_server_b200.models import DLRM, DLRMConfig, SyntheticCTR

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cfg = DLRMConfig()
    B = args.batch_per_gpu
    K, W = args.steps, args.warmup
    # every step may add up to B*26 new rows on the owners; size the index for the whole run
    capacity = max(1 << 22, (K * 2 + W + 8) * B * cfg.num_sparse * 2)
    if args.impl == "nccl_baseline":
        from parameter_server_b200.parallel import NcclDenseTable, NcclSparseTable
        model = DLRM(cfg, B, table_capacity=capacity, seed=0, sparse_cls=NcclSparseTable, dense_cls=NcclDenseTable)
        args.no_graph = True      # variable all-to-all split sizes need the host: not capturable
        args.no_sparse_micro = True
    else:
        model = DLRM(cfg, B, table_capacity=capacity, seed=0)
    data = SyntheticCTR(cfg, B, pool=16, seed=1000 + rank)
    uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
    uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid

    # ---------------- warm-up ----------------
    sampler = ClockSampler(uuid)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to come up: start it before the warm-up
    for _ in range(max(W, 3)):
        model.train_step(*data.next())
    model.check()
    own_launches_per_step = model.launches_per_step
    if not args.no_graph:
        model.enable_graph()
        for _ in range(3):
            model.train_step(*data.next())
        model.check()

    # ---------------- device-timed region ----------------
    sampler.mark()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(K):
        model.train_step(*data.next())
    ev1.record()
    barrier()
    ms = max_over_ranks(ev0.elapsed_time(ev1))
    model.check()

    # ---------------- end-to-end region (public API, loss read back every step) ----------------
    barrier()
    ev0.record()
    t0 = time.perf_counter()
    last_loss = 0.0
    for _ in range(K):
        model.train_step(*data.next())
        last_loss = model.read_loss()
    ev1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(ev0.elapsed_time(ev1), wall_ms))
    clocks = sampler.stop() if rank == 0 else None
    model.check()

    samples = B * world * K
    value = samples / (ms / 1e3)
    e2e_value = samples / (e2e_ms / 1e3)
    keys_per_step = B * cfg.num_sparse * world
    result = {
        "metric": "dlrm_samples_per_sec",
        "value": value,
        "unit": "samples/s",
        "n_gpus": world,
        "steps": K,
        "warmup": max(W, 3),
        "ms_per_step": ms / K,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 MLP, fp32 embeddings + optimizer state",
        "data": "synthetic (Zipf(1.1) keys per field, log-normal dense, Bernoulli(0.03) labels), random-init weights",
        "impl": args.impl,
        "config": {
            "model": "DLRM 13 dense + 26 sparse fields, emb dim 128 fp32 Adagrad on the PS, bottom 13-512-256-128, "
                     "27x128 pairwise-dot interaction, top 1024-1024-512-256-1 bf16 AdamW on the PS, BCE",
            "global_batch": B * world,
            "batch_per_gpu": B,
            "seq_len": None,
            "parallelism": f"dp{world} + sparse rows sharded by key hash + dense slices (PS)",
            "vocab": "26 fields log-spaced 1e3..4e7 (~300M rows), rows created on first pull",
            "launch": "eager" if args.no_graph else "whole step replayed from one CUDA graph",
            "l2": "inputs larger than L2: ~109 MB of embedding rows gathered + ~109 MB of row gradients per step "
                  "per GPU, new batch (pool of 16) every step",
        },
        "clocks": clocks,
        "e2e": {
            "value": e2e_value,
            "unit": "samples/s",
            "ms_per_step": e2e_ms / K,
            "h2d_bytes_per_step": data.bytes_per_batch(),
            "d2h_bytes_per_step": 4,
            "last_loss": last_loss,
        },
        "gpu_launches": own_launches_per_step * K,
        "sparse_keys_per_step": keys_per_step,
        "sparse_pull_push_keys_per_sec_in_step": 2 * keys_per_step * K / (ms / 1e3),
        "table_rows_rank0": model.sparse.size(),
    }
    if args.breakdown and hasattr(model, "step_breakdown"):
        barrier()
        result["breakdown_us_rank0"] = model.step_breakdown()
        barrier()
    if args.impl == "nccl_baseline":
        result["config"]["parallelism"] = f"dp{world} + NCCL all_to_all_single sparse path + reduce_scatter/all_gather dense path (baseline)"

    # ---------------- sparse pull+push microbenchmark (config 2 shape, dim 64 + Adagrad) ----------------
    if not args.no_sparse_micro:
        del model
        torch.cuda.empty_cache()
        result["sparse_micro"] = sparse_micro(args, world, rank, barrier, max_over_ranks)

    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def sparse_micro(args, world, rank, barrier, max_over_ranks) -> dict:
    """Pull+push key throughput: dim 64 fp32 + Adagrad slot, Zipf(1.05) keys with at least 30% in-batch
    duplicates, ``--micro-keys`` keys per GPU per step. Device-timed, max over ranks."""
    import numpy as np
    import torch

    from parameter_server_b200 import SparseTable
    from parameter_server_b200.utils.keys import zipf_batch

    n = args.micro_keys
    steps, warm = 20, 5
    t = SparseTable(64, "adagrad", dict(lr=0.05, init_accumulator=0.1), capacity=(steps + warm + 2) * n,
                    max_keys=n, seed=3)
    rng = np.random.default_rng(77 + rank)
    pool = []
    for _ in range(8):
        k = zipf_batch(rng, n, 1.05, 500_000_000 * world // 8 + 1, 0.3)
        pool.append(torch.from_numpy(k).cuda())
    grads = torch.randn(n, 64, device="cuda") * 1e-3
    out = torch.empty(n, 64, device="cuda")
    for i in range(warm):
        t.pull(pool[i % 8], out=out)
        t.push(grads)
    t.check()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    barrier()
    pull_ms = push_ms = 0.0
    e[0].record()
    for i in range(steps):
        t.pull(pool[i % 8], out=out)
        t.push(grads)
    e[1].record()
    barrier()
    both_ms = max_over_ranks(e[0].elapsed_time(e[1]))
    # pull alone / push alone
    barrier()
    e[0].record()
    for i in range(steps):
        t.pull(pool[i % 8], out=out)
    e[1].record()
    barrier()
    pull_ms = max_over_ranks(e[0].elapsed_time(e[1]))
    t.check()
    uniq = t.engine.last_unique(0)
    total = n * world * steps
    return {
        "keys_per_gpu_per_step": n, "dim": 64, "optimizer": "adagrad", "zipf_s": 1.05,
        "unique_fraction_last_batch": uniq / n,
        "pull_push_keys_per_sec": 2 * total / (both_ms / 1e3),
        "pull_keys_per_sec": total / (pull_ms / 1e3),
        "ms_per_pull_push": both_ms / steps, "ms_per_pull": pull_ms / steps,
        "table_rows_rank0": t.size(),
    }


if __name__ == "__main__":
    main()
