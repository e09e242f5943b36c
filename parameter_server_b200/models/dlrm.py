"""DLRM-style CTR model trained against the parameter server.

Embeddings live in a :class:`SparseTable` (fused pull in the forward pass, fused push of the row
gradients in the backward pass); the MLP weights live in a :class:`DenseTable` (fused
reduce-scatter + optimizer + all-gather). The dense math is hand-written sm_100a code: the tcgen05
GEMM for every linear layer (forward, dgrad with the ReLU mask in the epilogue, split-K wgrad), the
pairwise-dot interaction and the output layer fused with sigmoid + BCE. The forward and backward
passes are written out explicitly (no autograd graph), with all activations preallocated, so a
step is a fixed sequence of kernel launches.

The reference ships no model code; this is the consumer that its sparse + dense operators are built
for (config 3 of the benchmark: 13 dense features, 26 sparse fields, embedding dim 128, bottom MLP
13-512-256-128, 27x128 pairwise-dot interaction, top MLP 1024-1024-512-256-1, BCE loss).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from .._lib import C
from ..ops import gemm as G
from ..ops.dense import DenseTable
from ..ops.sparse import SparseTable, _stream


@dataclass
class DLRMConfig:
    num_dense: int = 13
    num_sparse: int = 26
    emb_dim: int = 128
    bottom: Sequence[int] = (512, 256, 128)
    top: Sequence[int] = (1024, 1024, 512, 256)
    vocab_min: float = 1e3
    vocab_max: float = 4e7
    zipf_s: float = 1.1
    label_rate: float = 0.03
    sparse_optimizer: str = "adagrad"
    sparse_opt_kwargs: dict = field(default_factory=lambda: dict(lr=0.05, init_accumulator=0.1))
    dense_optimizer: str = "adamw"
    dense_opt_kwargs: dict = field(default_factory=lambda: dict(lr=1e-3, weight_decay=0.0))

    def vocab_sizes(self) -> List[int]:
        return [int(round(v)) for v in np.logspace(np.log10(self.vocab_min), np.log10(self.vocab_max), self.num_sparse)]


def _pad8(v: int) -> int:
    return (v + 7) // 8 * 8


def _pad64(v: int) -> int:
    return (v + 63) // 64 * 64


def field_keys(field_ids: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Globally unique int64 key of (field, id): the field index in the bits above 2^40."""
    return (field_ids.to(torch.int64) << 40) | ids.to(torch.int64)


class SyntheticCTR:
    """Synthetic click data of the benchmark shape: log-normal dense features, per-field Zipf keys,
    Bernoulli labels. Batches are generated on the host into pinned memory (the input pipeline of a
    real job ends there), ``pool`` of them are kept and cycled."""

    def __init__(self, cfg: DLRMConfig, batch: int, pool: int = 8, seed: int = 0, pin: bool = True):
        rng = np.random.default_rng(seed)
        vocab = np.array(cfg.vocab_sizes(), dtype=np.int64)
        self.batches = []
        fid = np.arange(cfg.num_sparse, dtype=np.int64)[None, :] << 40
        for _ in range(pool):
            dense = rng.lognormal(0.0, 1.0, size=(batch, cfg.num_dense)).astype(np.float32)
            z = rng.zipf(cfg.zipf_s, size=(batch, cfg.num_sparse)).astype(np.int64)
            ids = (z - 1) % vocab[None, :]
            keys = fid | ids
            labels = (rng.random(batch) < cfg.label_rate).astype(np.float32)
            t = (torch.from_numpy(dense), torch.from_numpy(keys), torch.from_numpy(labels))
            if pin and torch.cuda.is_available():
                t = tuple(x.pin_memory() for x in t)
            self.batches.append(t)
        self.i = 0

    def next(self):
        b = self.batches[self.i % len(self.batches)]
        self.i += 1
        return b

    def bytes_per_batch(self) -> int:
        return sum(x.numel() * x.element_size() for x in self.batches[0])


class DLRM:
    """One rank's replica of the model; ``train_step`` is collective over the ranks of ``group``."""

    def __init__(self, cfg: DLRMConfig, batch: int, *, table_capacity: int = 1 << 22, device=None, group=None,
                 seed: int = 0, wgrad_split_k: int = 0, sparse_kwargs: Optional[dict] = None,
                 sparse_cls=SparseTable, dense_cls=DenseTable, overlap: Optional[bool] = None, pull_sms: int = 124,
                 push_sms: int = 96, chain_gemms: bool = True, grad_wire_bf16: bool = True,
                 tail_overlap: Optional[bool] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("DLRM runs on the sm_100a kernels and needs a CUDA device")
        self.cfg = cfg
        self.B = batch
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.group = group
        D, F = cfg.emb_dim, cfg.num_sparse
        assert cfg.bottom[-1] == D, "bottom MLP must end at the embedding width"
        self.split_k = wgrad_split_k
        # sparse_cls / dense_cls let the NCCL-only baseline tables stand in for the fused ones
        self.sparse = sparse_cls(D, cfg.sparse_optimizer, cfg.sparse_opt_kwargs, capacity=table_capacity,
                                  max_keys=batch * F, device=self.device, group=group, seed=seed,
                                  **(sparse_kwargs or {}))
        # ---- dense parameters ------------------------------------------------------------------
        self.k_in = _pad8(cfg.num_dense)
        n_inter = D + (F + 1) * F // 2
        # the interaction output is padded to whole 64-column blocks (zero columns, zero weight columns): the GEMMs
        # that read it transposed (dgrad, wgrad) then fetch each operand stage with one bulk-tensor load
        self.k_top = _pad64(n_inter)
        self.n_inter = n_inter
        bdims = [self.k_in] + list(cfg.bottom)
        tdims = [self.k_top] + list(cfg.top)
        shapes = {}
        for i in range(len(bdims) - 1):
            shapes[f"bot.w{i}"] = (bdims[i + 1], bdims[i])
            shapes[f"bot.b{i}"] = (bdims[i + 1],)
        for i in range(len(tdims) - 1):
            shapes[f"top.w{i}"] = (tdims[i + 1], tdims[i])
            shapes[f"top.b{i}"] = (tdims[i + 1],)
        shapes["head.w"] = (tdims[-1],)
        shapes["head.b"] = (1,)
        self.dense = dense_cls(shapes, cfg.dense_optimizer, cfg.dense_opt_kwargs, grad_dtype=torch.float32,
                                device=self.device, group=group)
        gen = torch.Generator().manual_seed(seed + 1)
        init = {}
        for name, shape in shapes.items():
            if ".w" in name and len(shape) == 2:
                fan_in = shape[1]
                w = torch.randn(shape, generator=gen) * (2.0 / fan_in) ** 0.5
                if name == "bot.w0":
                    w[:, cfg.num_dense:] = 0
                if name == "top.w0":
                    w[:, n_inter:] = 0
                init[name] = w
            elif name == "head.w":
                init[name] = torch.randn(shape, generator=gen) * (1.0 / shape[0]) ** 0.5
            else:
                init[name] = torch.zeros(shape)
        self.dense.load(init)
        self.bdims, self.tdims = bdims, tdims
        # ---- preallocated activations --------------------------------------------------------------
        dev, bf = self.device, torch.bfloat16
        B = batch
        # Two sets of input buffers: while step t computes on one set, the host -> device copy of batch t + 1 lands in
        # the other (a copy stream of its own), so the PCIe transfer is off the critical path of the step.
        self._inputs = [(torch.empty((B, cfg.num_dense), dtype=torch.float32, device=dev),
                         torch.empty((B, F), dtype=torch.int64, device=dev),
                         torch.empty((B,), dtype=torch.float32, device=dev)) for _ in range(2)]
        self._slot = 0
        self._staged = None   # input-buffer set holding a batch that no step has consumed yet
        self.d_dense, self.d_keys, self.d_labels = self._inputs[0]
        self.copy_stream = torch.cuda.Stream(device=dev)
        self._in_ready = [torch.cuda.Event() for _ in range(2)]
        self._in_consumed = [torch.cuda.Event() for _ in range(2)]
        self.x16 = torch.empty((B, self.k_in), dtype=bf, device=dev)
        self.bot_act = [torch.empty((B, n), dtype=bf, device=dev) for n in cfg.bottom]
        # the pull delivers the embedding rows in the dtype their consumer (the interaction kernels) computes in
        self.emb_bf16 = bool(getattr(self.sparse, "supports_bf16_out", False))
        self.emb = torch.empty((B * F, D), dtype=bf if self.emb_bf16 else torch.float32, device=dev)
        self.inter = torch.empty((B, self.k_top), dtype=bf, device=dev)
        self.top_act = [torch.empty((B, n), dtype=bf, device=dev) for n in cfg.top]
        self.top_dz = [torch.empty((B, n), dtype=bf, device=dev) for n in cfg.top]
        self.d_inter = torch.empty((B, self.k_top), dtype=bf, device=dev)
        self.bot_dz = [torch.empty((B, n), dtype=bf, device=dev) for n in cfg.bottom]
        self.d_emb = torch.empty((B * F, D), dtype=torch.float32, device=dev)
        self.loss = torch.zeros(1, dtype=torch.float32, device=dev)
        self.h_loss = torch.zeros(1, dtype=torch.float32).pin_memory()
        self.launches_per_step = 0
        # the layers of each MLP pass (bottom forward, top forward, top dgrad, bottom dgrad) run as one chained launch
        self.chain_gemms = bool(chain_gemms)
        # Overlap: the sparse pull runs on a side stream beside the bottom MLP forward, the sparse push beside the
        # bottom dgrad + weight / bias gradients. The GPU is shared by SMs: a CTA of the fused sparse kernels and a
        # CTA of the GEMM each fill an SM, so the pull (push) is launched on ``pull_sms`` (``push_sms``) SMs and the
        # GEMMs of the concurrent branch on the others, whichever kernel happens to start first.
        # Measured on B200: the split pays on one GPU (about 5 % of the step) and on two (2 %); from four ranks on the
        # pull and push spend much of their time waiting for peers, and SMs held by a waiting kernel are lost to the
        # GEMMs, so the default (None) turns the overlap on for up to two ranks only.
        # ``overlap="fwd"``: only the pull runs beside the bottom MLP; the backward pass keeps one stream (plus the tail
        # arrangement below).
        if overlap is None:
            overlap = getattr(self.sparse, "world", 1) <= 2
        can_split = hasattr(self.sparse, "set_sm_budget")
        self.overlap_fwd = (overlap == "fwd" or overlap is True) and can_split
        self.overlap = (overlap is True) and can_split
        self.n_sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.pull_sms = max(8, min(int(pull_sms), self.n_sms - 8))
        self.push_sms = max(8, min(int(push_sms), self.n_sms - 8))
        # From three ranks on another pairing pays instead: the two kernels that wait for peers, the sparse push and the
        # dense push, run side by side at the end of the step (the sparse push on all SMs but `dense_sms`, the dense
        # push, which is small, on those), so the waits of the dense push hide under the sparse push.
        self.dense_sms = 16
        want_tail = (getattr(self.sparse, "world", 1) > 2) if tail_overlap is None else bool(tail_overlap)
        self.tail_overlap = (not self.overlap) and want_tail and hasattr(self.sparse, "set_sm_budget") and \
            hasattr(self.dense, "set_sm_budget")
        if self.overlap or self.overlap_fwd or self.tail_overlap:
            self.side = torch.cuda.Stream(device=dev)
            self.sparse.set_sm_budget(self.pull_sms if self.overlap_fwd else 0,
                                      self.push_sms if self.overlap else (self.n_sms - self.dense_sms if self.tail_overlap else 0))
        if self.tail_overlap:
            self.dense.set_sm_budget(self.dense_sms)
        # the row gradients come out of bf16 tensor-core arithmetic; between ranks they travel as bf16 like the rows
        if grad_wire_bf16 and hasattr(self.sparse, "set_grad_wire_bf16"):
            self.sparse.set_grad_wire_bf16(True)
        self.graph = None
        self.graphs = [None, None]   # one captured step per input-buffer set
        self.trace = None   # list of (section, CUDA event) while a step is being traced
        self.stamps = None  # device buffer of %globaltimer probes while a traced graph is being captured

    # ------------------------------------------------------------------------------------------
    def load_batch(self, dense: torch.Tensor, keys: torch.Tensor, labels: torch.Tensor) -> None:
        """Host (pinned) -> device copies of one batch on the current stream."""
        self.d_dense.copy_(dense, non_blocking=True)
        self.d_keys.copy_(keys, non_blocking=True)
        self.d_labels.copy_(labels, non_blocking=True)

    def _mark(self, name: str) -> None:
        if self.trace is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.trace.append((name, e))
        if self.stamps is not None:
            # a one-thread kernel writes %globaltimer when the current stream gets here (works inside a graph)
            i = len(self.stamp_names)
            self.stamp_names.append(name + ("@side" if torch.cuda.current_stream() != self._main_stream else ""))
            C.timestamp(self.stamps[i:].data_ptr(), _stream())

    def graph_timeline(self, repeats: int = 20) -> dict:
        """Where the time goes inside the captured step: the step is captured once more with one-thread timestamp
        kernels between its sections (on the main stream, and around the pull / push on the side stream), replayed
        ``repeats`` times on the batch in the input buffers, and the median time of every probe since the first one is
        returned in microseconds (probes of the side stream are marked ``@side``). Each probe adds a launch of about
        2 us to its stream, so the last offset is a little above the plain step."""
        import statistics
        self.stamps = torch.zeros(64, dtype=torch.int64, device=self.device)
        self.stamp_names = []
        self._main_stream = None
        self.sparse.reserve(4 * self.sparse.world * self.B * self.cfg.num_sparse)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._main_stream = torch.cuda.current_stream()
            self._mark("start")
            self.forward_backward()
        names = list(self.stamp_names)
        runs = []
        for _ in range(repeats):
            g.replay()
            torch.cuda.synchronize()
            runs.append(self.stamps[:len(names)].tolist())
        self.stamps = None
        # offset of every probe from the first one, median over the replays
        out = {nm: round(statistics.median((r[i] - r[0]) / 1e3 for r in runs), 1) for i, nm in enumerate(names) if i > 0}
        return out

    def step_breakdown(self, repeats: int = 5) -> dict:
        """Device time of each section of the step in microseconds (median over ``repeats`` eager steps on
        the batch in the input buffers), plus the in-kernel phase times of the fused sparse pull / push.
        Sections that wait for other ranks include the skew between the ranks."""
        import statistics
        acc: dict = {}
        cta_spread: dict = {}
        prof = getattr(self.sparse, "engine", None)
        if prof is not None and hasattr(prof, "set_profile"):
            prof.set_profile(True)
        for _ in range(repeats):
            self.trace = []
            self._mark("start")
            self.forward_backward()
            torch.cuda.synchronize()
            for (_, e0), (name, e1) in zip(self.trace, self.trace[1:]):
                acc.setdefault(name, []).append(e0.elapsed_time(e1) * 1e3)
            if prof is not None and hasattr(prof, "phase_stamps"):
                st = prof.phase_stamps(0)
                for i, nm in enumerate(["pull.P1_dedup", "pull.P2_ship_keys", "pull.P3a_resolve", "pull.P3b_init", "pull.P3c_rows",
                                        "pull.P5_gather"]):
                    acc.setdefault(nm, []).append((st[i + 1] - st[i]) / 1e3)
                if self.sparse.world > 1:
                    spans = [(8, 9, "push.Q1_segsum_ack_wait"), (9, 10, "push.Q2_ship_wait_grads"), (10, 11, "push.Q3ab_elect_fold"),
                             (11, 12, "push.Q3c_update")]
                else:   # a single rank has no ship phase and leaves stamp 9 unwritten
                    spans = [(8, 10, "push.Q1_segsum"), (10, 11, "push.Q3ab_elect_fold"), (11, 12, "push.Q3c_update")]
                for lo, hi, nm in spans:
                    acc.setdefault(nm, []).append((st[hi] - st[lo]) / 1e3)
                if hasattr(prof, "cta_stamps"):
                    # when each CTA reached the barrier that ends a phase, relative to the phase's start in CTA 0
                    t_in = [x for x in prof.cta_stamps(0, 0) if x]
                    for which, ref, nm in ((1, st[0], "pull.P1_cta_arrival"), (2, st[2], "pull.P3a_cta_arrival"),
                                           (3, st[8], "push.Q1_cta_arrival")):
                        v = sorted((x - ref) / 1e3 for x in prof.cta_stamps(which, 0) if x)
                        if v:
                            cta_spread[nm] = [round(v[0], 1), round(v[len(v) // 2], 1), round(v[-1], 1)]
                    if t_in:
                        cta_spread["pull.cta_start_spread"] = [0.0, round((sorted(t_in)[len(t_in) // 2] - min(t_in)) / 1e3, 1),
                                                               round((max(t_in) - min(t_in)) / 1e3, 1)]
        self.trace = None
        if prof is not None and hasattr(prof, "set_profile"):
            prof.set_profile(False)
        out = {k: round(statistics.median(v), 1) for k, v in acc.items()}
        if prof is not None and hasattr(prof, "last_unique"):
            # distinct keys of this rank's last pull, and the time their rows need on one NVLink direction
            # (770 GB/s measured peer copy): the floor of the row-return phase of the pull and of the gradient
            # shipment of the push when there is more than one rank
            uniq = int(prof.last_unique(0))
            w = self.sparse.world
            out["unique_keys_last_pull"] = uniq
            out["remote_row_bytes"] = int(uniq * (w - 1) / w * self.cfg.emb_dim * 4)
            out["nvlink_floor_us_per_direction"] = round(out["remote_row_bytes"] / 770e9 * 1e6, 1)
        if cta_spread:
            out["cta_us_min_median_max"] = cta_spread
        return out

    def forward_backward(self) -> torch.Tensor:
        """One training step on the batch already in the device input buffers. Returns the device
        loss tensor (mean BCE over this rank's batch)."""
        cfg, B, D, F = self.cfg, self.B, self.cfg.emb_dim, self.cfg.num_sparse
        P, Gd = self.dense.params, self.dense.grads
        s = _stream()
        n_launch = 0

        def chk(rc):
            if rc != 0:
                raise RuntimeError(f"kernel launch failed: {rc}")

        # ---------------- forward ----------------
        main = torch.cuda.current_stream()
        if self.overlap_fwd:
            # fork: the pull needs only the keys; it runs beside the dense-feature cast and the bottom MLP
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                self.sparse.pull(self.d_keys, out=self.emb); n_launch += 1
                if self.stamps is not None:
                    self._mark("pull_done")
            # the GEMMs beside the pull: single CTAs (a pair needs two free SMs of one TPC) on the other SMs
            C.gemm_set_cta_limit(self.n_sms - self.pull_sms)
            C.gemm_set_pair(0)
        self.dense.zero_grads()  # torch fill kernels (not counted as own launches)
        self.loss.zero_()
        chk(C.cast_pad(self.d_dense.data_ptr(), B, cfg.num_dense, self.x16.data_ptr(), self.k_in, s)); n_launch += 1
        self._mark("zero_cast")
        n_launch += self._mlp_forward(self.x16, self.bot_act, "bot")
        self._mark("bottom_fwd")
        if self.overlap_fwd:
            C.gemm_set_cta_limit(0)
            C.gemm_set_pair(1)
            main.wait_stream(self.side)   # join: the interaction needs the embedding rows
        else:
            self.sparse.pull(self.d_keys, out=self.emb); n_launch += 1
        self._mark("sparse_pull")
        chk(C.interaction_fwd(self.bot_act[-1].data_ptr(), D, self.emb.data_ptr(), F, D, self.inter.data_ptr(),
                              self.k_top, B, s, self.emb_bf16)); n_launch += 1
        self._mark("interaction_fwd")
        n_launch += self._mlp_forward(self.inter, self.top_act, "top")
        self._mark("top_fwd")
        # ---------------- head: logits + loss + first backward step ----------------
        last = len(self.top_act) - 1
        chk(C.bce_head(self.top_act[last].data_ptr(), self.tdims[-1], P["head.w"].data_ptr(), P["head.b"].data_ptr(),
                       self.d_labels.data_ptr(), B, self.tdims[-1], 1.0 / B, self.loss.data_ptr(), 0,
                       self.top_dz[last].data_ptr(), self.tdims[-1], Gd["head.w"].data_ptr(), Gd["head.b"].data_ptr(), s))
        n_launch += 1
        self._mark("head")
        # ---------------- backward: the dgrad chain first; every layer's dz stays in its own buffer, so the
        # weight and bias gradients of ALL layers run at the end as one grouped GEMM launch (two when a layer
        # is too narrow for the wide tile) and one bias-gradient launch ----------------
        wg, bg = [], []
        dgrad = []
        for i in range(last, -1, -1):
            dz = self.top_dz[i]
            x_in = self.top_act[i - 1] if i > 0 else self.inter
            wg.append((dz, x_in, Gd[f"top.w{i}"]))
            bg.append((dz, Gd[f"top.b{i}"]))
            if i > 0:
                dgrad.append(dict(a=dz, w=P[f"top.w{i}"], mask=self.top_act[i - 1], out=self.top_dz[i - 1]))
            else:
                dgrad.append(dict(a=dz, w=P["top.w0"], out=self.d_inter))
        n_launch += self._dgrad_chain(dgrad)
        self._mark("top_bwd")
        # ---------------- backward: interaction + sparse push ----------------
        nb = len(self.bot_act) - 1
        chk(C.interaction_bwd(self.d_inter.data_ptr(), self.k_top, self.bot_act[nb].data_ptr(), D, self.emb.data_ptr(),
                              F, D, self.bot_dz[nb].data_ptr(), D, self.d_emb.data_ptr(), B, True, s, self.emb_bf16)); n_launch += 1
        self._mark("interaction_bwd")
        if self.overlap:
            # fork: the push needs only the row gradients; the rest of the backward pass does not need the push
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                self.sparse.push(self.d_emb); n_launch += 1
                if self.stamps is not None:
                    self._mark("push_done")
            C.gemm_set_cta_limit(self.n_sms - self.push_sms)
            C.gemm_set_pair(0)
        elif not self.tail_overlap:
            self.sparse.push(self.d_emb); n_launch += 1
        self._mark("sparse_push")
        # ---------------- backward: bottom MLP ----------------
        dgrad = []
        for i in range(nb, -1, -1):
            dz = self.bot_dz[i]
            x_in = self.bot_act[i - 1] if i > 0 else self.x16
            wg.append((dz, x_in, Gd[f"bot.w{i}"]))
            bg.append((dz, Gd[f"bot.b{i}"]))
            if i > 0:
                dgrad.append(dict(a=dz, w=P[f"bot.w{i}"], mask=self.bot_act[i - 1], out=self.bot_dz[i - 1]))
        n_launch += self._dgrad_chain(dgrad)
        self._mark("bottom_dgrad")
        G.grouped_wgrad(wg, split_k=self.split_k)
        n_launch += (1 if any(x.shape[1] >= 256 for _, x, _ in wg) else 0) + (1 if any(x.shape[1] < 256 for _, x, _ in wg) else 0)
        self._mark("wgrad")
        G.bias_grads(bg); n_launch += (len(bg) + 7) // 8
        self._mark("bias_grad")
        if self.overlap:
            C.gemm_set_cta_limit(0)
            C.gemm_set_pair(1)
            # join before the dense push: it waits for the other ranks like the sparse push does, and two kernels
            # that wait for peers must not compete for the same SMs
            main.wait_stream(self.side)
            self._mark("join_push")
        if self.tail_overlap:
            # fork: the sparse push beside the dense push; both wait for their peers, on disjoint SMs
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                self.sparse.push(self.d_emb); n_launch += 1
                if self.stamps is not None:
                    self._mark("push_done")
        self.dense.push(); n_launch += 1
        if self.tail_overlap:
            main.wait_stream(self.side)
        self._mark("dense_push")
        self.launches_per_step = n_launch
        return self.loss

    def _mlp_forward(self, x: torch.Tensor, acts, prefix: str) -> int:
        """``acts[i] = relu(acts[i-1] @ W_i^T + b_i)``; returns the number of launches."""
        P = self.dense.params
        layers = []
        a = x
        for i, out in enumerate(acts):
            layers.append(dict(a=a, w=P[f"{prefix}.w{i}"], bias=P[f"{prefix}.b{i}"], relu=True, out=out))
            a = out
        if self.chain_gemms:
            G.chain(layers)
            return 1
        for l in layers:
            G.gemm(l["a"], l["w"], bias=l["bias"], relu=True, out=l["out"])
        return len(layers)

    def _dgrad_chain(self, layers) -> int:
        """``dz_{i-1} = (dz_i @ W_i) * (act_{i-1} > 0)`` down an MLP; returns the number of launches."""
        if not layers:
            return 0
        if self.chain_gemms:
            G.chain(layers, b_mn=True)
            return 1
        for l in layers:
            G.linear_dgrad(l["a"], l["w"], mask=l.get("mask"), out=l["out"])
        return len(layers)

    def _use_slot(self, slot: int) -> None:
        self._slot = slot
        self.d_dense, self.d_keys, self.d_labels = self._inputs[slot]

    def enable_graph(self) -> None:
        """Capture the step (every launch of ``forward_backward``) in a CUDA graph, once per input-buffer set; later
        ``train_step`` calls replay them in turn. Call after a few eager steps. What a captured launch cannot do
        moves out of it: row-pool growth happens on the host before each replay, the call epochs and
        the Adam step live in device memory and advance with every replay."""
        self.sparse.opt.step_from_epoch = 1
        self.dense.opt.step_from_epoch = 1
        self._worst_new_rows = self.sparse.world * self.B * self.cfg.num_sparse
        self.sparse.reserve(4 * self._worst_new_rows)
        torch.cuda.synchronize()
        keep = self._slot
        for slot in range(2):
            self._use_slot(slot)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.forward_backward()
            self.graphs[slot] = g
        self._use_slot(keep)
        self.graph = self.graphs[keep]

    def stage(self, dense: torch.Tensor, keys: torch.Tensor, labels: torch.Tensor) -> None:
        """Start the host -> device copy of the NEXT step's batch (pinned host tensors) on the copy stream, into the
        input-buffer set that the running step is not using. Called right after ``train_step`` it lets the transfer
        overlap the compute of the step just queued, also in a loop that reads the loss back after every step."""
        slot = self._slot ^ 1
        d_dense, d_keys, d_labels = self._inputs[slot]
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self._in_consumed[slot])   # the step that last read this set has finished
            d_dense.copy_(dense, non_blocking=True)
            d_keys.copy_(keys, non_blocking=True)
            d_labels.copy_(labels, non_blocking=True)
            self._in_ready[slot].record(self.copy_stream)
        self._staged = slot

    def train_step(self, dense: Optional[torch.Tensor] = None, keys: Optional[torch.Tensor] = None,
                   labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Public API: run one step and return the device loss. With a batch (pinned host tensors) the batch is
        staged first; without arguments the step runs on the batch handed to ``stage`` before. Either way the copy
        goes into the input-buffer set that the previous step is NOT using, on a copy stream: when the caller
        queues steps without waiting for each, or stages batch t + 1 before it reads the loss of step t, the
        transfer of batch t + 1 overlaps the compute of step t."""
        if dense is not None:
            self.stage(dense, keys, labels)
        if self._staged is None:
            raise RuntimeError("train_step() without a batch needs a stage(...) call before it")
        main = torch.cuda.current_stream()
        slot = self._staged
        self._staged = None
        self._use_slot(slot)
        main.wait_event(self._in_ready[slot])
        if self.graphs[slot] is None:
            out = self.forward_backward()
        else:
            self.sparse.reserve(self._worst_new_rows)
            self.graphs[slot].replay()
            out = self.loss
        self._in_consumed[slot].record(main)
        return out

    def read_loss(self) -> float:
        """Device -> host read of the last step's loss (synchronises the stream)."""
        self.h_loss.copy_(self.loss, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(self.h_loss.item())

    def check(self) -> None:
        self.sparse.check()
        self.dense.check()

    # ---- checkpoint / resume: the embedding table in the dump layout of the operator API, the MLPs with their
    # optimizer state as one slice per rank; both load on another number of ranks -------------------------------
    def save_checkpoint(self, uri: str, file_number: int = 1) -> None:
        """Collective, between steps. ``<uri>/sparse`` and ``<uri>/dense``."""
        from ..parallel import checkpoint
        torch.cuda.synchronize(self.device)
        checkpoint.dump(self.sparse, uri.rstrip("/") + "/sparse", file_number=file_number)
        checkpoint.dump_dense(self.dense, uri.rstrip("/") + "/dense")

    def load_checkpoint(self, uri: str) -> None:
        """Collective, between steps: the tables keep their buffers, so a captured step graph stays valid."""
        from ..parallel import checkpoint
        torch.cuda.synchronize(self.device)
        checkpoint.load(self.sparse, uri.rstrip("/") + "/sparse")
        checkpoint.load_dense(self.dense, uri.rstrip("/") + "/dense")
        G.check_gemm_errors()

    # ------------------------------------------------------------------------------------------
    def reference_loss(self) -> float:
        """Loss of the current device batch computed with plain fp32 PyTorch ops on the current
        parameters (read-only pull); used by the tests."""
        cfg, B, D, F = self.cfg, self.B, self.cfg.emb_dim, self.cfg.num_sparse
        P = {k: v.float() for k, v in self.dense.params.items()}
        x = torch.zeros((B, self.k_in), device=self.device)
        x[:, :cfg.num_dense] = self.d_dense
        x = x.bfloat16().float()
        for i in range(len(cfg.bottom)):
            x = torch.relu(x @ P[f"bot.w{i}"].t() + P[f"bot.b{i}"]).bfloat16().float()
        emb = self.sparse.pull(self.d_keys, insert=False, for_push=False).view(B, F, D)
        T = torch.cat([x[:, None, :], emb], dim=1)
        Z = torch.bmm(T, T.transpose(1, 2))
        ii, jj = torch.tril_indices(F + 1, F + 1, offset=-1)
        inter = torch.cat([x, Z[:, ii, jj]], dim=1)
        h = torch.zeros((B, self.k_top), device=self.device)
        h[:, :inter.shape[1]] = inter
        h = h.bfloat16().float()
        for i in range(len(cfg.top)):
            h = torch.relu(h @ P[f"top.w{i}"].t() + P[f"top.b{i}"]).bfloat16().float()
        z = h @ P["head.w"] + P["head.b"]
        return float(torch.nn.functional.binary_cross_entropy_with_logits(z, self.d_labels).item())
