"""All-gather fused into a GEMM (``ops.gemm.ag_linear``) against the unfused sequence on the same data:
NCCL ``all_gather_into_tensor`` of the weight shards followed by the plain GEMM. Run under torchrun, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m parameter_server_b200.utils.ag_bench --tokens 4096 --n 6144 --k 2048

Every rank holds the current values of its own N / world rows of W (a dense table with ``scatter_peers=False``, as
after a dense push that skips the all-gather half). Times: CUDA events on every rank after a barrier, max over ranks,
median over iterations; the L2 is flushed before every iteration. Dense pull fused with its first consumer:
pico-ps/operator/DensePullOperator.h:153-216.
"""
from __future__ import annotations

import argparse
import os
import statistics

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--gather-ctas", type=int, default=8)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    lr = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import gemm as G
    from ..ops.dense import DenseTable
    from .kernel_bench import flush_l2
    M, N, K = a.tokens, a.n, a.k
    table = DenseTable({"w": (N, K)}, "sgd", dict(lr=0.0), device=dev, scatter_peers=False)
    gen = torch.Generator().manual_seed(1)
    w_full = (torch.randn(N, K, generator=gen) * 0.05)
    table.load({"w": w_full})
    # only this rank's rows of its local copy are current: poison the others so that a missing gather shows
    rows = N // world
    W = table.params["w"]
    keep = W[rank * rows:(rank + 1) * rows].clone()
    W.fill_(float("nan"))
    W[rank * rows:(rank + 1) * rows] = keep
    shard = keep.contiguous()
    x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    out_f = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    out_u = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    w_all = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
    dist.barrier()
    torch.cuda.synchronize()

    def fused():
        # a fresh gather every call: the stale rows are poisoned again first (outside the timed region)
        G.ag_linear(x, table, "w", out=out_f, gather_ctas=a.gather_ctas)

    def unfused():
        dist.all_gather_into_tensor(w_all, shard)
        G.gemm(x, w_all, out=out_u)

    def gemm_only():
        G.gemm(x, w_all, out=out_u)

    def timed(fn, poison):
        ts = []
        for i in range(a.iters + 3):
            if poison:
                W.fill_(float("nan"))
                W[rank * rows:(rank + 1) * rows] = keep
            flush_l2()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if i >= 3:
                ts.append(float(t.item()))
        return statistics.median(ts) * 1e3

    t_f = timed(fused, True)
    G.check_gemm_errors()
    t_u = timed(unfused, False)
    t_g = timed(gemm_only, False)
    ok = torch.allclose(out_f.float(), out_u.float(), rtol=2e-2, atol=2e-2) and not torch.isnan(out_f.float()).any()
    oks = [None] * world
    dist.all_gather_object(oks, bool(ok))
    if rank == 0:
        remote = (world - 1) / world * N * K * 2
        print(f"ag_linear M={M} N={N} K={K} world={world}: fused {t_f:8.1f} us   all_gather + gemm {t_u:8.1f} us   gemm alone {t_g:8.1f} us")
        print(f"   remote weight bytes per rank {remote/1e6:.1f} MB = {remote/770e9*1e6:.1f} us at the 770 GB/s measured peer copy; "
              f"gather exposed in the fused launch {t_f - t_g:.1f} us, in the unfused sequence {t_u - t_g:.1f} us; results equal: {all(oks)}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
