#!/usr/bin/env python
"""Headline benchmark: DLRM-style CTR training against the parameter server (samples/s, whole job),
plus the sparse pull+push key throughput of the same kernels on a resident table.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|nccl_baseline] [--config dlrm|sparse]

For N > 1 the script is started once per GPU by ``python -m torch.distributed.run`` (it re-executes
itself that way when started plainly). Prints ONE JSON line on rank 0.

What is timed (own arm, ``--config dlrm``):
  value  device time (CUDA events, max over ranks) of K training steps, each including the
         host->device copy of that step's batch from pinned memory, the fused sparse pull, the
         tcgen05 MLP forward/backward, the fused sparse push and the fused dense push;
  e2e    the same K steps through the public calls ``DLRM.stage`` (host->device copy of a batch from pinned
         memory), ``DLRM.train_step`` and ``read_loss``: the loss of EVERY step is read back to the host
         (device->host) with a stream synchronisation before the next step is queued; the copy of batch
         k + 1 is started right after step k was queued, as a trainer with a one-batch-ahead input
         pipeline does. K copies and K reads lie inside the timed region.
  baseline / vs_baseline
         the reference publishes no number and cannot be built offline, so the same invocation then runs
         the same model, batch and steps on this repository's NCCL-only arm (torch.unique +
         all_to_all_single + library index ops for the sparse path, reduce_scatter + all_gather for
         the dense path) and ``vs_baseline`` = value / that arm's value.
Weak scaling: batch per GPU is fixed (global batch 65536 at 8 GPUs). Data is synthetic (per-field
Zipf keys, log-normal dense features, Bernoulli labels), weights are random-init, keys are new to the
table the first time they appear (pull inserts), so the table grows during the run.

``--config sparse`` runs benchmark config 2 alone: pull and pull+push key throughput on a resident table
swept over 64 Ki .. 4 Mi keys per GPU per step.
"""
from __future__ import annotations

import argparse
import gc
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
    ap.add_argument("--config", default="dlrm", choices=["dlrm", "sparse"],
                    help="dlrm: the CTR training step (config 3); sparse: the key-throughput sweep on a resident table (config 2)")
    ap.add_argument("--batch-per-gpu", type=int, default=8192)
    ap.add_argument("--no-sparse-micro", action="store_true", help="skip the sparse pull+push microbenchmark")
    ap.add_argument("--no-baseline", action="store_true", help="skip the NCCL-only arm (vs_baseline stays null)")
    ap.add_argument("--breakdown", action="store_true", help="after the timed regions, add per-section device times of an eager step")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-overlap", action="store_true", help="run the sparse pull / push in line with the dense work (one stream)")
    ap.add_argument("--overlap", action="store_true", help="force the side-stream overlap (default: on for up to two GPUs)")
    ap.add_argument("--overlap-fwd", action="store_true", help="only the pull beside the bottom MLP (the backward pass on one stream)")
    ap.add_argument("--no-tail-overlap", action="store_true", help="from 3 GPUs on: do not run the sparse push beside the dense push")
    ap.add_argument("--tail-overlap", action="store_true", help="run the sparse push beside the dense push at any number of GPUs (with --no-overlap)")
    ap.add_argument("--no-chain", action="store_true", help="one GEMM launch per MLP layer instead of one chained launch per MLP pass")
    ap.add_argument("--pull-sms", type=int, default=124, help="SMs of the fused sparse pull while it runs beside the bottom MLP (the GEMMs get the rest)")
    ap.add_argument("--push-sms", type=int, default=96, help="SMs of the fused sparse push while it runs beside the dense backward pass")
    ap.add_argument("--micro-keys", type=int, default=1 << 20, help="keys per GPU per step of the microbenchmark")
    ap.add_argument("--micro-rows", type=int, default=62_500_000, help="resident rows per GPU of the microbenchmark table (config 2: 500 M keys / 8)")
    ap.add_argument("--sizes", default="65536,262144,1048576,4194304", help="--config sparse: keys per GPU per step")
    return ap.parse_args()


class ClockSampler:
    """Samples the SM clock and the throttle reasons of this process's GPU during a region: through NVML in a
    thread (about one sample per millisecond, read-only queries), or through ``nvidia-smi`` when NVML cannot be
    loaded. ``start()`` returns once the first sample has arrived."""

    SMI_FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
                  "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                  "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str, period_s: float = 0.001):
        self.uuid = uuid
        self.period = period_s
        self.samples = []   # (sm_mhz, max_mhz, set of reason names)
        self.first = 0
        self.stop_flag = False
        self.thread = None
        self.proc = None
        self.how = None

    # ---- NVML --------------------------------------------------------------------------------------
    def _nvml_loop(self, nv, handle):
        # bit values of nvmlClocksEventReasons: SwPowerCap 0x4, HwSlowdown 0x8, SwThermalSlowdown 0x20, HwThermalSlowdown 0x40
        reasons = [("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4)]
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        smax = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
        while not self.stop_flag:
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM))
                mask = int(get_reasons(handle))
            except Exception:
                break
            self.samples.append((sm, smax, {name for name, bit in reasons if mask & bit}))
            time.sleep(self.period)

    def _start_nvml(self) -> bool:
        try:
            import pynvml as nv
            nv.nvmlInit()
        except Exception:
            return False
        handle = None
        for u in (self.uuid, self.uuid.encode()):   # the bindings of different versions take str or bytes
            try:
                handle = nv.nvmlDeviceGetHandleByUUID(u)
                break
            except Exception:
                continue
        if handle is None:
            return False
        self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
        self.thread.start()
        self.how = "nvml"
        return True

    # ---- nvidia-smi fallback -------------------------------------------------------------------------------
    def _smi_loop(self):
        for line in self.proc.stdout:
            p = [x.strip() for x in line.strip().split(",")]
            if len(p) < 8:
                continue
            try:
                sm, smax = float(p[0]), float(p[1])
            except ValueError:
                continue
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            self.samples.append((sm, smax, {n for n, v in zip(names, p[4:8]) if v.lower().startswith("active")}))

    def _start_smi(self) -> bool:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.SMI_FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return False
        self.thread = threading.Thread(target=self._smi_loop, daemon=True)
        self.thread.start()
        self.how = "nvidia-smi"
        return True

    def start(self, wait_s: float = 5.0) -> None:
        if not self._start_nvml() and not self._start_smi():
            return
        t0 = time.time()
        while not self.samples and time.time() - t0 < wait_s:   # block until the sampler delivers
            time.sleep(0.005)

    def mark(self) -> None:
        """Samples taken before this call (warm-up) are ignored by stop()."""
        self.first = len(self.samples)

    def stop(self) -> dict:
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        region = self.samples[self.first:] or self.samples
        if not region:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock sampler available"], "samples": 0}
        reasons = set()
        for _, _, r in region:
            reasons |= r
        return {"sm_mhz": statistics.median(s[0] for s in region), "sm_max_mhz": max(s[1] for s in region),
                "reasons": sorted(reasons), "samples": len(region), "sampler": self.how}


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

    def gather_clocks(c: dict) -> dict:
        """Every rank sampled its own GPU; rank 0 reports the slowest median, the union of the reasons and the
        smallest sample count."""
        if world == 1:
            return c
        allc = [None] * world
        dist.all_gather_object(allc, c)
        meds = [x["sm_mhz"] for x in allc if x.get("sm_mhz") is not None]
        return {"sm_mhz": min(meds) if meds else None,
                "sm_max_mhz": max((x["sm_max_mhz"] for x in allc if x.get("sm_max_mhz")), default=None),
                "reasons": sorted(set(r for x in allc for r in x.get("reasons", []))),
                "samples": min(x.get("samples", 0) for x in allc), "sampler": allc[0].get("sampler"),
                "per_rank_sm_mhz": [x.get("sm_mhz") for x in allc]}

    uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
    uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
    cfg = DLRMConfig()
    B = args.batch_per_gpu
    K, W = args.steps, max(args.warmup, 3)

    # ------------------------------------------------------------------------------------------------
    if args.config == "sparse":
        from parameter_server_b200.utils.sparse_bench import sweep
        sampler = ClockSampler(uuid)
        sampler.start()
        sampler.mark()
        res = sweep([int(s) for s in args.sizes.split(",")], args.micro_rows, "nccl" if args.impl == "nccl_baseline" else "ours",
                    64, max(K, 5), W, phases=args.breakdown)
        clocks = gather_clocks(sampler.stop())
        if rank == 0:
            top = max(res, key=lambda r: r["pull_push_keys_per_sec"])
            print(json.dumps({
                "metric": "sparse_pull_push_keys_per_sec", "value": top["pull_push_keys_per_sec"], "unit": "keys/s",
                "n_gpus": world, "steps": max(K, 5), "warmup": W, "ms_per_step": top["pull_push_ms"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 rows + Adagrad slot",
                "data": "synthetic Zipf(1.05) keys, >= 30 % duplicates per batch, random-init resident table",
                "impl": args.impl,
                "note": "value counts every key twice (one pull + one push = two key operations); "
                        "pull_push_steps_keys_per_sec in the sweep counts it once",
                "config": {"model": "sparse table dim 64 fp32 + Adagrad, %d resident rows per GPU" % args.micro_rows,
                           "global_batch": top["keys_per_gpu_per_step"] * world, "seq_len": None,
                           "parallelism": f"rows sharded by key hash over {world} GPU(s)",
                           "l2": "four key batches rotate; rows touched per step exceed L2 from 256 Ki keys up"},
                "clocks": clocks, "sweep": res}))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ------------------------------------------------------------------------------------------------
    def run_arm(impl: str, want_breakdown: bool) -> dict:
        """Builds the model for one arm, warms it up and times K steps twice (device-timed, then end to end)."""
        # every step may add up to B*26 new rows on the owners; size the index for the whole run
        capacity = max(1 << 22, (K * 2 + W + 8) * B * cfg.num_sparse * 2)
        graph = not args.no_graph
        if impl == "nccl_baseline":
            from parameter_server_b200.parallel import NcclDenseTable, NcclSparseTable
            model = DLRM(cfg, B, table_capacity=capacity, seed=0, sparse_cls=NcclSparseTable, dense_cls=NcclDenseTable,
                         chain_gemms=not args.no_chain)
            graph = False      # variable all-to-all split sizes need the host: not capturable
        else:
            model = DLRM(cfg, B, table_capacity=capacity, seed=0, overlap=(False if args.no_overlap else ("fwd" if args.overlap_fwd else (True if args.overlap else None))),
                         pull_sms=args.pull_sms, push_sms=args.push_sms, chain_gemms=not args.no_chain,
                         tail_overlap=(False if args.no_tail_overlap else (True if args.tail_overlap else None)))
        data = SyntheticCTR(cfg, B, pool=16, seed=1000 + rank)
        sampler = ClockSampler(uuid)
        sampler.start()          # returns once the first sample is in
        for _ in range(W):
            model.train_step(*data.next())
        model.check()
        launches = model.launches_per_step
        if graph:
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
        if hasattr(model, "stage"):
            # the loop of a trainer with a one-batch-ahead input pipeline: every step's inputs cross PCIe from pinned
            # memory inside the timed region (K copies), the copy of batch k + 1 is started right after step k was
            # queued, and the loss of every step is read back (synchronously) before the next step is queued
            model.stage(*data.next())
            for k in range(K):
                model.train_step()
                if k + 1 < K:
                    model.stage(*data.next())
                last_loss = model.read_loss()
        else:
            for _ in range(K):
                model.train_step(*data.next())
                last_loss = model.read_loss()
        ev1.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = max_over_ranks(max(ev0.elapsed_time(ev1), wall_ms))
        clocks = gather_clocks(sampler.stop())
        model.check()
        out = {"ms": ms, "e2e_ms": e2e_ms, "clocks": clocks, "launches": launches, "last_loss": last_loss,
               "h2d": data.bytes_per_batch(), "rows": model.sparse.size(), "graph": graph,
               "overlap": bool(getattr(model, "overlap", False)), "overlap_fwd": bool(getattr(model, "overlap_fwd", False)), "tail_overlap": bool(getattr(model, "tail_overlap", False))}
        if want_breakdown and hasattr(model, "step_breakdown"):
            barrier()
            out["breakdown"] = model.step_breakdown()
            barrier()
            if world == 1 and hasattr(model, "graph_timeline"):
                out["graph_timeline_us"] = model.graph_timeline()
        del model, data
        gc.collect()
        torch.cuda.empty_cache()
        return out

    own = run_arm(args.impl, args.breakdown)
    samples = B * world * K
    value = samples / (own["ms"] / 1e3)
    e2e_value = samples / (own["e2e_ms"] / 1e3)
    keys_per_step = B * cfg.num_sparse * world
    result = {
        "metric": "dlrm_samples_per_sec",
        "value": value,
        "unit": "samples/s",
        "n_gpus": world,
        "steps": K,
        "warmup": W,
        "ms_per_step": own["ms"] / K,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 MLP; fp32 embedding rows + optimizer state, fp32 sums; rows and row gradients cross NVLink as bf16",
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
            "launch": "whole step replayed from one CUDA graph" if own["graph"] else "eager",
            "streams": ("sparse pull beside the bottom MLP forward and sparse push beside bottom dgrad + weight / bias "
                        "gradients (side stream; the GPU is split by SMs: pull %d / push %d SMs, GEMMs on the rest)" % (args.pull_sms, args.push_sms)) if own["overlap"] else (
                            ("pull beside the bottom MLP (%d SMs / rest); " % args.pull_sms if own.get("overlap_fwd") else "one stream; ") +
                            ("the sparse push (all SMs but 16) and the dense push (16 SMs) run side by side" if own.get("tail_overlap") else "")),
            "l2": "inputs larger than L2: ~55 MB of bf16 embedding rows gathered + ~109 MB of fp32 row gradients per step "
                  "per GPU, new batch (pool of 16) every step",
        },
        "clocks": own["clocks"],
        "e2e": {
            "value": e2e_value,
            "unit": "samples/s",
            "ms_per_step": own["e2e_ms"] / K,
            "h2d_bytes_per_step": own["h2d"],
            "d2h_bytes_per_step": 4,
            "last_loss": own["last_loss"],
        },
        "gpu_launches": own["launches"] * K,
        "sparse_keys_per_step": keys_per_step,
        # every key of a step is pulled once and pushed once: two key operations per key
        "sparse_key_ops_per_sec_in_step": 2 * keys_per_step * K / (own["ms"] / 1e3),
        "sparse_keys_per_sec_in_step": keys_per_step * K / (own["ms"] / 1e3),
        "table_rows_rank0": own["rows"],
    }
    if "breakdown" in own:
        result["breakdown_us_rank0"] = own["breakdown"]
    if "graph_timeline_us" in own:
        result["graph_timeline_us"] = own["graph_timeline_us"]
    if args.impl == "nccl_baseline":
        result["config"]["parallelism"] = f"dp{world} + NCCL all_to_all_single sparse path + reduce_scatter/all_gather dense path (baseline)"

    # ---------------- the baseline the driver can see: the NCCL-only arm, same invocation ----------------
    if args.impl == "ours" and not args.no_baseline:
        try:
            base = run_arm("nccl_baseline", False)
            b_value = samples / (base["ms"] / 1e3)
            b_e2e = samples / (base["e2e_ms"] / 1e3)
            result["baseline"] = {
                "what": "this repository's NCCL-only arm (torch.unique + all_to_all_single + index ops; reduce_scatter + "
                        "torch AdamW + all_gather), same model, batch, steps and timing; the reference publishes no number "
                        "and cannot be built offline",
                "value": b_value, "ms_per_step": base["ms"] / K, "e2e_value": b_e2e, "e2e_ms_per_step": base["e2e_ms"] / K,
                "clocks": base["clocks"], "last_loss": base["last_loss"],
            }
            result["vs_baseline"] = value / b_value
            result["e2e"]["vs_baseline"] = e2e_value / b_e2e
        except Exception as ex:   # the baseline must never take the headline down with it
            result["baseline"] = {"error": repr(ex)[:300]}

    # ---------------- sparse pull+push microbenchmark (config 2 shape, dim 64 + Adagrad) ----------------
    if not args.no_sparse_micro and args.impl == "ours":
        from parameter_server_b200.utils.sparse_bench import sweep
        t0 = time.time()
        r = sweep([args.micro_keys], args.micro_rows, "ours", 64, 20, 5)[0]
        result["sparse_micro"] = {
            "keys_per_gpu_per_step": r["keys_per_gpu_per_step"], "dim": 64, "optimizer": "adagrad", "zipf_s": 1.05,
            "resident_rows_per_gpu": r["table_rows_max_per_gpu"], "table_keys": r["table_keys"],
            "unique_fraction": r["unique_fraction"],
            "ms_per_pull": r["pull_ms"], "ms_per_pull_push": r["pull_push_ms"],
            "pull_keys_per_sec": r["pull_keys_per_sec"],
            "pull_push_steps_keys_per_sec": r["pull_push_steps_keys_per_sec"],
            "pull_push_keys_per_sec": r["pull_push_keys_per_sec"],
            "counting": "pull_push_keys_per_sec counts every key twice (a pull and a push are two key operations); "
                        "pull_push_steps_keys_per_sec counts it once",
            "pull_push_algorithmic_gbs_per_gpu": r["pull_push_algorithmic_gbs_per_gpu"],
            "wall_s_including_table_build": round(time.time() - t0, 1),
        }

    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
