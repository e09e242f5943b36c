"""Micro-benchmarks of the hand-written kernels, one workload per sub-command.

    python -m parameter_server_b200.utils.kernel_bench gemm --m 8192 --n 1024 --k 1024
    python -m parameter_server_b200.utils.kernel_bench sparse --keys 1048576 --dim 64 --zipf 1.05
    python -m parameter_server_b200.utils.kernel_bench interaction --batch 8192
    python -m parameter_server_b200.utils.kernel_bench dense --numel 67108864

Timing: CUDA events on the launching stream, >= 3 warm-up iterations, L2 flushed between timed
iterations (a 256 MB buffer is overwritten), median over the iterations. Each line reports the achieved
rate and its fraction of the measured roofline (``MEASURED_PEAKS.json`` at the repository root when
present, else 6.65 TB/s and 1.59 PFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return j["hbm_gbs"] * 1e9, j["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


def timed(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return statistics.median(ts)


def cmd_gemm(a):
    from ..ops import gemm as G
    hbm, flops_peak, src = peaks()
    M, N, K = a.m, a.n, a.k
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    dy = torch.randn(M, N, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(N, K, device="cuda")
    cases = {
        "fwd  y=xW^T (K,K)": lambda: G.gemm(x, w, out=out),
        "dgrad dx=dyW (K,MN)": lambda: G.gemm(dy, w, b_mn=True, out=dx),
        "wgrad dW=dy^Tx (MN,MN)": lambda: G.linear_wgrad(dy, x, out=dw, split_k=0),
    }
    fl = 2.0 * M * N * K
    for name, fn in cases.items():
        if a.only and a.only not in name:
            continue
        t = timed(fn, a.iters, flush=not a.no_flush)
        print(f"gemm {name:24s} M={M} N={N} K={K}: {t*1e6:8.1f} us  {fl/t/1e12:7.1f} TFLOP/s  "
              f"{fl/t/flops_peak:5.2f} of {src} bf16 peak")
    if a.cublas:
        t = timed(lambda: torch.matmul(x, w.t(), out=out), a.iters, flush=not a.no_flush)
        print(f"gemm torch.matmul (cuBLAS) reference      : {t*1e6:8.1f} us  {fl/t/1e12:7.1f} TFLOP/s")
    G.check_gemm_errors()


def cmd_sparse(a):
    from ..ops.sparse import SparseTable
    hbm, _, src = peaks()
    n, dim = a.keys, a.dim
    t = SparseTable(dim, "adagrad", dict(lr=0.05, init_accumulator=0.1), capacity=4 * n, max_keys=n)
    rng = np.random.default_rng(0)
    pool = []
    for _ in range(4):
        k = rng.zipf(a.zipf, size=n).astype(np.uint64) if a.zipf > 1 else rng.integers(0, a.vocab, size=n).astype(np.uint64)
        k = ((k * np.uint64(0x9E3779B97F4A7C15)) >> np.uint64(2)) % np.uint64(a.vocab)
        pool.append(torch.from_numpy(k.astype(np.int64)).cuda())
    grads = torch.randn(n, dim, device="cuda") * 1e-3
    out = torch.empty(n, dim, device="cuda")
    if a.deterministic:
        t.set_deterministic(True)
    if a.sms:
        t.set_sm_budget(a.sms, a.sms)
    t.reserve(8 * n, exact=True)
    for i in range(8):
        t.pull(pool[i % 4], out=out)
        t.push(grads)
    t.check()
    it = [0]

    def pull():
        t.pull(pool[it[0] % 4], out=out)
        it[0] += 1

    tp = timed(pull, a.iters, flush=not a.no_flush)
    uniq = t.engine.last_unique(0)

    def both():
        t.pull(pool[it[0] % 4], out=out)
        t.push(grads)
        it[0] += 1

    tb = timed(both, a.iters, flush=not a.no_flush)
    t.check()
    row = dim * 4
    stride = row * 2
    pull_bytes = uniq * row + n * row + n * 8
    push_bytes = n * row + uniq * (2 * stride)
    print(f"sparse pull  n={n} dim={dim} unique={uniq/n:.2f}: {tp*1e6:8.1f} us  {n/tp/1e9:6.2f} Gkeys/s  "
          f"algorithmic {pull_bytes/tp/1e9:7.0f} GB/s = {pull_bytes/tp/hbm:4.2f} of {src} HBM copy")
    print(f"sparse pull+push               : {tb*1e6:8.1f} us  {2*n/tb/1e9:6.2f} Gkeys/s  "
          f"algorithmic {(pull_bytes+push_bytes)/tb/1e9:7.0f} GB/s = {(pull_bytes+push_bytes)/tb/hbm:4.2f} of {src} HBM copy")
    if a.phases:
        t.engine.set_profile(True)
        both()
        st = t.engine.phase_stamps(0)
        names = ["P1 dedup", "P2 ship", "P3a resolve", "P3b init", "P3c rows", "P5 gather"]
        for i, nm in enumerate(names):
            print(f"   {nm:12s} {(st[i+1]-st[i])/1e3:8.1f} us")
        print(f"   {'Q1 segsum':12s} {(st[10]-st[8])/1e3:8.1f} us  (CTA 0: chain + cache set-up {(st[13]-st[8])/1e3:.1f}, sums {(st[14]-st[13])/1e3:.1f}, "
              f"cache flush {(st[15]-st[14])/1e3:.1f}, barrier {(st[10]-st[15])/1e3:.1f})")
        v = sorted((x - st[8]) / 1e3 for x in t.engine.cta_stamps(3, 0) if x)
        if v:
            print(f"   Q1 CTA arrival at the barrier: min {v[0]:.1f}  median {v[len(v)//2]:.1f}  max {v[-1]:.1f} us")
        print(f"   {'Q3c update':12s} {(st[12]-st[11])/1e3:8.1f} us")


def cmd_interaction(a):
    from .._lib import C
    hbm, _, src = peaks()
    B, F, D, ldo = a.batch, 26, 128, 480
    bottom = torch.randn(B, D, device="cuda").bfloat16()
    emb = torch.randn(B, F, D, device="cuda") * 0.1
    out = torch.empty(B, ldo, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn(B, ldo, device="cuda").bfloat16()
    dbot = torch.empty(B, D, device="cuda", dtype=torch.bfloat16)
    demb = torch.empty(B, F, D, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    tf = timed(lambda: C.interaction_fwd(bottom.data_ptr(), D, emb.data_ptr(), F, D, out.data_ptr(), ldo, B, s), a.iters)
    tb = timed(lambda: C.interaction_bwd(dout.data_ptr(), ldo, bottom.data_ptr(), D, emb.data_ptr(), F, D, dbot.data_ptr(), D,
                                         demb.data_ptr(), B, True, s), a.iters)
    fb = B * (F * D * 4 + D * 2 + ldo * 2)
    bb = B * (2 * F * D * 4 + 2 * D * 2 + ldo * 2)
    print(f"interaction fwd B={B}: {tf*1e6:7.1f} us  {fb/tf/1e9:6.0f} GB/s = {fb/tf/hbm:4.2f} of {src} HBM copy")
    print(f"interaction bwd B={B}: {tb*1e6:7.1f} us  {bb/tb/1e9:6.0f} GB/s = {bb/tb/hbm:4.2f} of {src} HBM copy")


def cmd_dense(a):
    from ..ops.dense import DenseTable
    hbm, _, src = peaks()
    t = DenseTable({"w": (a.numel,)}, "adamw", dict(lr=1e-3), grad_dtype=torch.bfloat16 if a.bf16_grads else torch.float32)
    t.load({"w": torch.zeros(a.numel)})
    t.flat_grads.fill_(1e-3)
    tt = timed(lambda: t.push(), a.iters)
    t.check()
    gb = 2 if a.bf16_grads else 4
    bytes_ = a.numel * (gb + 3 * 4 * 2 + 2)   # grads read, master/m/v read+write, bf16 params written
    print(f"dense push (optimizer + bf16 write, world 1) numel={a.numel}: {tt*1e6:8.1f} us  {bytes_/tt/1e9:6.0f} GB/s = "
          f"{bytes_/tt/hbm:4.2f} of {src} HBM copy")


def graph_timed(fn, iters=20):
    """Median device time of ``fn`` replayed from a CUDA graph (no host launch gaps), L2 flushed before each replay."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return statistics.median(ts)


def cmd_mlp(a):
    """The MLP passes of the DLRM step (batch rows x layer widths): one launch per layer, one chained launch for the
    whole pass, and torch.matmul (cuBLAS, without the bias / ReLU epilogues) for reference. Graph replays."""
    from ..ops import gemm as G
    _, flops_peak, src = peaks()
    M = a.batch
    for name, dims in (("top forward", (512, 1024, 1024, 512, 256)), ("bottom forward", (16, 512, 256, 128))):
        ws = [(torch.randn(dims[i + 1], dims[i], device="cuda") * (2.0 / dims[i]) ** 0.5).bfloat16() for i in range(len(dims) - 1)]
        bs = [(torch.randn(dims[i + 1], device="cuda") * 0.1).bfloat16() for i in range(len(dims) - 1)]
        x = torch.randn(M, dims[0], device="cuda").bfloat16()
        outs = [torch.empty(M, d, device="cuda", dtype=torch.bfloat16) for d in dims[1:]]
        layers, prev = [], x
        for w, b, o in zip(ws, bs, outs):
            layers.append(dict(a=prev, w=w, bias=b, relu=True, out=o))
            prev = o

        def separate():
            for l in layers:
                G.gemm(l["a"], l["w"], bias=l["bias"], relu=True, out=l["out"])

        def chained():
            G.chain(layers)

        def cublas():
            for l in layers:
                torch.matmul(l["a"], l["w"].t(), out=l["out"])

        fl = sum(2.0 * M * dims[i] * dims[i + 1] for i in range(len(dims) - 1))
        for tag, fn in (("one launch per layer", separate), ("one chained launch", chained), ("torch.matmul per layer", cublas)):
            t = graph_timed(fn, a.iters)
            print(f"mlp {name:15s} M={M} {tag:24s}: {t*1e6:8.1f} us  {fl/t/1e12:7.1f} TFLOP/s  {fl/t/flops_peak:5.2f} of {src} bf16 peak")
        for i, l in enumerate(layers):
            t = graph_timed(lambda: G.gemm(l["a"], l["w"], bias=l["bias"], relu=True, out=l["out"]), a.iters)
            t2 = graph_timed(lambda: torch.matmul(l["a"], l["w"].t(), out=l["out"]), a.iters)
            f1 = 2.0 * M * dims[i] * dims[i + 1]
            print(f"    layer {i} [{M} x {dims[i + 1]} x {dims[i]}]: {t*1e6:7.1f} us ({f1/t/1e12:6.1f} TFLOP/s)   cuBLAS {t2*1e6:7.1f} us")
    # ---- backward: the dgrad chain of the top MLP and the grouped weight gradients of all layers ----
    dims = (256, 512, 1024, 1024, 512)          # dz widths walking down the top MLP
    ws = [(torch.randn(dims[i], dims[i + 1], device="cuda") * 0.05).bfloat16() for i in range(len(dims) - 1)]   # [k][n]
    masks = [torch.randn(M, dims[i + 1], device="cuda").bfloat16() for i in range(len(dims) - 2)] + [None]
    dz = torch.randn(M, dims[0], device="cuda").bfloat16()
    outs = [torch.empty(M, d, device="cuda", dtype=torch.bfloat16) for d in dims[1:]]
    layers, prev = [], dz
    for w, m, o in zip(ws, masks, outs):
        layers.append(dict(a=prev, w=w, mask=m, out=o))
        prev = o
    fl = sum(2.0 * M * dims[i] * dims[i + 1] for i in range(len(dims) - 1))

    def d_separate():
        for l in layers:
            G.linear_dgrad(l["a"], l["w"], mask=l["mask"], out=l["out"])

    def d_cublas():
        for l in layers:
            torch.matmul(l["a"], l["w"], out=l["out"])

    for tag, fn in (("one launch per layer", d_separate), ("one chained launch", lambda: G.chain(layers, b_mn=True)),
                    ("torch.matmul per layer", d_cublas)):
        t = graph_timed(fn, a.iters)
        print(f"mlp top dgrad       M={M} {tag:24s}: {t*1e6:8.1f} us  {fl/t/1e12:7.1f} TFLOP/s  {fl/t/flops_peak:5.2f} of {src} bf16 peak")
    shapes = [(1024, 512), (1024, 1024), (512, 1024), (256, 512), (256, 512), (128, 256)]    # (N_out, K_in) of the wide layers
    items, fl = [], 0.0
    for n_out, k_in in shapes:
        items.append(((torch.randn(M, n_out, device="cuda") * 0.5).bfloat16(), (torch.randn(M, k_in, device="cuda") * 0.5).bfloat16(),
                      torch.zeros(n_out, k_in, device="cuda")))
        fl += 2.0 * M * n_out * k_in

    def w_cublas():
        for dy, x, out in items:
            torch.matmul(dy.t(), x, out=out.bfloat16() if False else None)

    for tag, fn in (("grouped, one launch", lambda: G.grouped_wgrad(items)),
                    ("one launch per layer", lambda: [G.linear_wgrad(dy, x, out=out, split_k=0) for dy, x, out in items]),
                    ("torch.matmul per layer", w_cublas)):
        t = graph_timed(fn, a.iters)
        print(f"mlp wgrad (6 layers) M={M} {tag:24s}: {t*1e6:8.1f} us  {fl/t/1e12:7.1f} TFLOP/s  {fl/t/flops_peak:5.2f} of {src} bf16 peak")
    G.check_gemm_errors()


def cmd_chain(a):
    """One MLP pass of the DLRM step as the model launches it (eager launches, for a profiler): ``top_fwd`` and
    ``top_dgrad`` are one chained launch each, ``wgrad`` is the grouped weight-gradient launch."""
    from ..ops import gemm as G
    M = a.batch
    if a.which == "wgrad":
        shapes = [(1024, 512), (1024, 1024), (512, 1024), (256, 512), (256, 512), (128, 256)]
        items = [((torch.randn(M, n, device="cuda") * 0.5).bfloat16(), (torch.randn(M, k, device="cuda") * 0.5).bfloat16(),
                  torch.zeros(n, k, device="cuda")) for n, k in shapes]
        fn = lambda: G.grouped_wgrad(items)
        fl = sum(2.0 * M * n * k for n, k in shapes)
    else:
        fwd = a.which == "top_fwd"
        dims = (512, 1024, 1024, 512, 256) if fwd else (256, 512, 1024, 1024, 512)
        if fwd:
            ws = [(torch.randn(dims[i + 1], dims[i], device="cuda") * 0.05).bfloat16() for i in range(4)]
        else:
            ws = [(torch.randn(dims[i], dims[i + 1], device="cuda") * 0.05).bfloat16() for i in range(4)]
        bs = [(torch.randn(dims[i + 1], device="cuda") * 0.1).bfloat16() for i in range(4)]
        masks = [torch.randn(M, dims[i + 1], device="cuda").bfloat16() for i in range(3)] + [None]
        x = torch.randn(M, dims[0], device="cuda").bfloat16()
        outs = [torch.empty(M, d, device="cuda", dtype=torch.bfloat16) for d in dims[1:]]
        layers, prev = [], x
        for i in range(4):
            layers.append(dict(a=prev, w=ws[i], bias=bs[i], relu=True, out=outs[i]) if fwd else dict(a=prev, w=ws[i], mask=masks[i], out=outs[i]))
            prev = outs[i]
        fn = lambda: G.chain(layers, b_mn=not fwd)
        fl = sum(2.0 * M * dims[i] * dims[i + 1] for i in range(4))
    t = timed(fn, a.iters, flush=not a.no_flush)
    G.check_gemm_errors()
    print(f"chain {a.which} M={M}: {t*1e6:8.1f} us (eager launch, CUDA events)  {fl/t/1e12:7.1f} TFLOP/s")
    if a.trace:
        # per-unit timeline of CTA 0 (ns since its first stamp): where a tile's time goes
        from .._lib import C
        buf = torch.zeros(256, dtype=torch.int64, device="cuda")
        C.gemm_set_trace(buf.data_ptr())
        if not a.no_flush:
            flush_l2()
        fn()
        torch.cuda.synchronize()
        C.gemm_set_trace(0)
        v = buf.view(8, 32).tolist()
        t0 = min(r[0] for r in v if r[0])
        names = ["load0", "loadN", "mma0", "data0", "commit", "epi_w0", "epi_all", "tmem0", "math0", "smem0", "stage0", "issue0", "epi_end"]
        order = [0, 1, 2, 3, 4, 8, 5, 9, 15, 16, 10, 11, 6]
        print(" unit " + " ".join(f"{n:>8s}" for n in names) + "   (ns after CTA 0's first load)")
        for r in v:
            if r[0]:
                mhz = (r[21] - r[20]) / max(1, r[4] - r[3]) * 1e3
                print(f"{r[7]:5d} " + " ".join(f"{(r[k] - t0) if r[k] else -1:8d}" for k in order) + f"   SM clock {mhz:6.0f} MHz")


def cmd_scaling(a):
    """How the GEMM launches of the DLRM step and the fused sparse kernels scale with the SMs they get: the input to
    the choice of the SM split when the two run side by side (``DLRM(overlap=True, pull_sms=, push_sms=)``)."""
    import contextlib
    import io
    from .._lib import C
    from ..ops.sparse import SparseTable
    n_sms = torch.cuda.get_device_properties(0).multi_processor_count
    for lim in (0, 112, 74, 36):
        C.gemm_set_cta_limit(lim)
        C.gemm_set_pair(0 if lim else 1)
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            cmd_mlp(a)
        print(f"== GEMM launches on {lim or n_sms} SMs" + ("" if lim else " (CTA pairs)"))
        for ln in buf.getvalue().splitlines():
            if "chained" in ln or "grouped" in ln:
                print(ln)
    C.gemm_set_cta_limit(0)
    C.gemm_set_pair(1)
    # a DLRM-like batch: 26 fields, Zipf(1.1) per field, vocabularies log-spaced 1e3 .. 4e7, dim 128
    B, F, dim = a.batch, 26, 128
    rng = np.random.default_rng(0)
    vocab = np.logspace(3, np.log10(4e7), F).astype(np.int64)

    def batch():
        ks = [(rng.zipf(1.1, size=B).astype(np.int64) % vocab[f]) + (np.int64(f) << np.int64(40)) for f in range(F)]
        return torch.from_numpy(np.stack(ks, 1).reshape(-1)).cuda()

    n = B * F
    t = SparseTable(dim, "adagrad", dict(lr=0.05, init_accumulator=0.1), capacity=8 * n, max_keys=n)
    pool = [batch() for _ in range(8)]
    grads = torch.randn(n, dim, device="cuda") * 1e-3
    out = torch.empty(n, dim, device="cuda", dtype=torch.bfloat16)
    t.reserve(8 * n, exact=True)
    for i in range(16):
        t.pull(pool[i % 8], out=out)
        t.push(grads)
    t.check()
    it = [0]

    def pull():
        t.pull(pool[it[0] % 8], out=out)
        it[0] += 1

    def both():
        pull()
        t.push(grads)

    for sms in (0, 148, 112, 90, 74, 37):
        if sms > n_sms:
            continue
        t.set_sm_budget(sms, sms)
        tp = timed(pull, a.iters)
        tb = timed(both, a.iters)
        t.check()
        shape = f"{sms} SMs, 1024-thread CTAs" if sms else f"{n_sms} SMs, 256-thread CTAs x 4"
        print(f"sparse pull / push of {n} keys, dim {dim}, on {shape}: pull {tp*1e6:7.1f} us   push {(tb-tp)*1e6:7.1f} us")


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192); g.add_argument("--n", type=int, default=1024); g.add_argument("--k", type=int, default=1024)
    g.add_argument("--only", default=""); g.add_argument("--cublas", action="store_true")
    s = sub.add_parser("sparse")
    s.add_argument("--keys", type=int, default=1 << 20); s.add_argument("--dim", type=int, default=64)
    s.add_argument("--zipf", type=float, default=1.05); s.add_argument("--vocab", type=int, default=62_500_000)
    s.add_argument("--phases", action="store_true")
    s.add_argument("--deterministic", action="store_true", help="reproducible pushes (sorted segment sum)")
    s.add_argument("--sms", type=int, default=0, help="SM budget of pull and push (0 = whole GPU, 256-thread CTAs)")
    i = sub.add_parser("interaction")
    i.add_argument("--batch", type=int, default=8192)
    d = sub.add_parser("dense")
    d.add_argument("--numel", type=int, default=64 << 20); d.add_argument("--bf16-grads", action="store_true")
    m = sub.add_parser("mlp")
    m.add_argument("--batch", type=int, default=8192)
    c = sub.add_parser("chain")
    c.add_argument("--which", default="top_fwd", choices=["top_fwd", "top_dgrad", "wgrad"])
    c.add_argument("--batch", type=int, default=8192)
    c.add_argument("--trace", action="store_true", help="print the per-tile timeline of CTA 0")
    sc = sub.add_parser("scaling")
    sc.add_argument("--batch", type=int, default=8192)
    for p in (g, s, i, d, m, c, sc):
        p.add_argument("--iters", type=int, default=10)
        p.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()
    {"gemm": cmd_gemm, "sparse": cmd_sparse, "interaction": cmd_interaction, "dense": cmd_dense, "mlp": cmd_mlp, "chain": cmd_chain,
     "scaling": cmd_scaling}[a.cmd](a)


if __name__ == "__main__":
    main()
