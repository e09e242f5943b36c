"""bf16 GEMM on tcgen05 / TMEM / TMA (``csrc/kernels/gemm_tcgen05.cu``) and the linear-layer triple
built on it (forward, dgrad, wgrad) without transposed copies."""
from __future__ import annotations

from typing import Optional

import torch

from .._lib import C

_err_flags = {}


def _err_flag(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _err_flags:
        _err_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err_flags[key]


def check_gemm_errors(device=None) -> None:
    """Synchronise and raise if a bounded wait inside a GEMM kernel ran out."""
    for key, flag in _err_flags.items():
        v = int(flag.item())
        if v:
            flag.zero_()
            raise RuntimeError(f"tcgen05 GEMM on cuda:{key}: bounded wait ran out (site {v})")


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, bias: Optional[torch.Tensor] = None,
         relu: bool = False, mask: Optional[torch.Tensor] = None, accumulate: bool = False, split_k: int = 1,
         M: Optional[int] = None, N: Optional[int] = None, K: Optional[int] = None, gather: Optional[dict] = None,
         wait_limit_s: float = 2.0) -> torch.Tensor:
    """``out[M,N] = epilogue(sum_k A(m,k) B(n,k))``.

    ``a`` is ``[M,K]`` (or ``[K,M]`` with ``a_mn``), ``b`` is ``[N,K]`` (or ``[K,N]`` with ``b_mn``);
    both bf16, row-major (last stride 1, leading dimension a multiple of 8).
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda and b.is_cuda
    assert a.stride(-1) == 1 and b.stride(-1) == 1
    if M is None:
        M = a.shape[1] if a_mn else a.shape[0]
    if K is None:
        K = a.shape[0] if a_mn else a.shape[1]
    if N is None:
        N = b.shape[1] if b_mn else b.shape[0]
    # the kernel reads and writes what M, N, K say: they must lie inside the tensors that were handed in
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("gemm operands are 2-D")
    am, ak = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    bn, bk = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if M > am or K > ak or N > bn or K > bk:
        raise ValueError(f"gemm: M, N, K = {M}, {N}, {K} exceed the operands ({am} x {ak} and {bn} x {bk})")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    elif not out.is_cuda or out.dim() != 2 or out.shape[0] < M or out.shape[1] < N:
        raise ValueError(f"gemm: out must be a CUDA tensor of at least {M} x {N}")
    if bias is not None and (not bias.is_cuda or bias.numel() < N):
        raise ValueError(f"gemm: bias must be a CUDA tensor of at least {N} elements")
    if mask is not None and (not mask.is_cuda or mask.dim() != 2 or mask.shape[0] < M or mask.shape[1] < N):
        raise ValueError(f"gemm: mask must be a CUDA tensor of at least {M} x {N}")
    assert out.stride(-1) == 1
    o16 = out if out.dtype == torch.bfloat16 else None
    o32 = out if out.dtype == torch.float32 else None
    assert o16 is not None or o32 is not None
    b32 = bias if (bias is not None and bias.dtype == torch.float32) else None
    b16 = bias if (bias is not None and bias.dtype == torch.bfloat16) else None
    if split_k > 1:
        assert o32 is not None and o16 is None, "split-K accumulates into a zero-initialised fp32 output"
    rc = C.gemm_bf16(a.data_ptr(), a.stride(0), a_mn, b.data_ptr(), b.stride(0), b_mn, M, N, K,
                     _ptr(o16), _ptr(o32), out.stride(0), _ptr(b32), relu, _ptr(mask),
                     mask.stride(0) if mask is not None else 0, accumulate, _ptr(b16), split_k,
                     _err_flag(a.device).data_ptr(), wait_limit_s,
                     torch.cuda.current_stream().cuda_stream, **(gather or {}))
    if rc != 0:
        raise RuntimeError(f"gemm_bf16 failed with code {rc}")
    return out


def linear_fwd(x, w, bias=None, relu=False, out=None):
    """y = act(x @ w.T + bias); x [M,K], w [N,K]."""
    return gemm(x, w, bias=bias, relu=relu, out=out)


def linear_dgrad(dy, w, mask=None, out=None):
    """dx = (dy @ w) * (mask > 0); dy [M,N], w [N,K] -> dx [M,K]."""
    return gemm(dy, w, b_mn=True, mask=mask, out=out)


def linear_wgrad(dy, x, out=None, accumulate=False, split_k=1):
    """dw = dy.T @ x; dy [M,N], x [M,K] -> dw [N,K] fp32. With ``split_k`` > 1 the batch dimension is
    split over CTAs and ``out`` must be zero-initialised (partials are added atomically)."""
    if split_k <= 0:  # automatic: enough K slices to give every SM a tile
        n_out, k_in, batch = dy.shape[1], x.shape[1], dy.shape[0]
        bn = 256 if k_in >= 256 else 128
        tiles = ((n_out + 127) // 128) * ((k_in + bn - 1) // bn)
        split_k = max(1, min(16, 148 // tiles, max(1, batch // 256)))
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, out_dtype=torch.float32, accumulate=accumulate,
                split_k=split_k)


_chain_scratch = {}


def chain(layers, *, b_mn: bool = False, wait_limit_s: float = 2.0) -> None:
    """The layers of an MLP (forward: ``b_mn=False``, ``w`` is ``[N, K]``; dgrad: ``b_mn=True``, ``w`` is ``[K, N]``) in
    ONE persistent launch. ``layers`` is a list of dicts ``a, w, out`` (+ ``bias`` bf16, ``relu``, ``mask``); layer
    ``i + 1`` must read ``out`` of layer ``i`` as its ``a``. Inside the kernel the next layer starts on a row block as
    soon as the previous layer has stored it, so no layer pays a launch, a ramp-up or a drained tail of its own."""
    if not 1 <= len(layers) <= 8:
        raise ValueError("a chain holds 1..8 layers")
    dev = layers[0]["a"].device
    stream = torch.cuda.current_stream().cuda_stream
    key = (dev.index or 0, stream)
    if key not in _chain_scratch:
        _chain_scratch[key] = torch.zeros(C.gemm_chain_scratch_words(), dtype=torch.int32, device=dev)
    probs = []
    for i, l in enumerate(layers):
        a, w, out = l["a"], l["w"], l["out"]
        bias, mask = l.get("bias"), l.get("mask")
        assert a.dtype == w.dtype == out.dtype == torch.bfloat16 and a.stride(-1) == w.stride(-1) == out.stride(-1) == 1
        assert bias is None or bias.dtype == torch.bfloat16
        M, K = a.shape
        N = w.shape[1] if b_mn else w.shape[0]
        assert (w.shape[0] if b_mn else w.shape[1]) == K and out.shape[0] == M and out.shape[1] >= N
        if i > 0:
            assert a.data_ptr() == layers[i - 1]["out"].data_ptr(), "layer i + 1 must read the output of layer i"
        probs.append((a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), M, N, K, out.data_ptr(), out.stride(0),
                      _ptr(bias), bool(l.get("relu", False)), _ptr(mask), mask.stride(0) if mask is not None else 0))
    rc = C.gemm_bf16_chain(probs, b_mn, _chain_scratch[key].data_ptr(), _err_flag(dev).data_ptr(), wait_limit_s, stream)
    if rc != 0:
        raise RuntimeError(f"gemm_bf16_chain failed with code {rc}")


def grouped_wgrad(items, split_k: int = 0) -> None:
    """Weight gradients of several linear layers in as few launches as possible. ``items`` is a list of
    ``(dy, x, out)`` with ``dy [M, N_i]``, ``x [M, K_i]`` bf16 and ``out [N_i, K_i]`` fp32, zero-initialised (the
    batch dimension is split over CTAs and partial sums are added atomically). Layers whose input width fills a
    256-wide tile share one persistent launch, the narrow ones another: the small problems of an MLP fill the
    machine together instead of each paying its own ramp-up and tail."""
    wide = [it for it in items if it[1].shape[1] >= 256]
    narrow = [it for it in items if it[1].shape[1] < 256]
    for group, bn in ((wide, 256), (narrow, 128)):
        for lo in range(0, len(group), 8):
            part = group[lo:lo + 8]
            batch = part[0][0].shape[0]
            tiles = sum(((dy.shape[1] + 127) // 128) * ((x.shape[1] + bn - 1) // bn) for dy, x, _ in part)
            sk = split_k
            if sk <= 0:   # about two waves of work units over the 148 SMs, at least 8 k-tiles per unit
                sk = max(1, min(16, round(296 / tiles), max(1, batch // 512)))
            probs = []
            for dy, x, out in part:
                assert dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and out.dtype == torch.float32
                assert dy.stride(-1) == 1 and x.stride(-1) == 1 and out.stride(-1) == 1 and dy.shape[0] == x.shape[0]
                probs.append((dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), dy.shape[1], x.shape[1], dy.shape[0],
                              0, out.data_ptr(), out.stride(0), False, sk))
            rc = C.gemm_bf16_grouped(probs, True, True, _err_flag(part[0][0].device).data_ptr(), 2.0,
                                     torch.cuda.current_stream().cuda_stream)
            if rc != 0:
                raise RuntimeError(f"gemm_bf16_grouped failed with code {rc}")


def bias_grads(items) -> None:
    """``db_i += dz_i.sum(0)`` for a list of ``(dz, db)`` (bf16 ``[M, N_i]``, fp32 ``[N_i]``) in one launch per 8."""
    for lo in range(0, len(items), 8):
        part = items[lo:lo + 8]
        rc = C.bias_grad_multi([(dz.data_ptr(), dz.stride(0), dz.shape[1], db.data_ptr()) for dz, db in part],
                               part[0][0].shape[0], torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"bias_grad_multi failed: {rc}")


def ag_linear(x: torch.Tensor, table, name: str, *, bias=None, relu: bool = False, out=None, gather_ctas: int = 8) -> torch.Tensor:
    """``y = act(x @ W.T + bias)`` where ``W = table[name]`` is a dense-table tensor whose rows are sharded over the
    ranks and whose peer copies are NOT kept current by the dense push (``DenseTable(scatter_peers=False)``):
    the all-gather of W is fused into this GEMM. The first ``gather_ctas`` CTAs pull the remote row blocks over
    NVLink into the local copy while the other CTAs already multiply the local rows; a tile of remote rows
    waits for its block's flag. Dense pull fused with its first consumer
    (pico-ps/operator/DensePullOperator.h:153-169,197-216)."""
    W = table.params[name]
    N, K = W.shape
    world, rank = table.world, table.rank
    if world == 1:
        return gemm(x, W, bias=bias, relu=relu, out=out)
    off, _ = table.offsets[name]
    if off != 0 or table.numel != N * K or N % (256 * world):
        raise ValueError("ag_linear needs a dense table that holds exactly this tensor, rows divisible by 256 * world")
    if table._ag_ready is None:
        table._ag_ready = torch.zeros(N // 256, dtype=torch.int32, device=W.device)
    table._ag_epoch += 1
    g = dict(gather_peers=[table.engine.peer_params_ptr(r) for r in range(world)], gather_rank=rank,
             rows_per_rank=N // world, gather_ready=table._ag_ready.data_ptr(), gather_epoch=table._ag_epoch,
             gather_ctas=gather_ctas)
    return gemm(x, W, bias=bias, relu=relu, out=out, gather=g)
