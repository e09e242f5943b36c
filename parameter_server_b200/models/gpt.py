"""GPT-style decoder trained with its dense parameters on the parameter server.

Config 4 of the benchmark: 24 layers, d_model 2048, 16 heads, FFN 8192, vocab 50304, sequence 2048, bf16,
data parallel over the GPUs of one box. Every linear layer runs on the tcgen05 GEMM (forward, dgrad,
wgrad accumulating in fp32 straight into the dense table's gradient buffer). Dense push = the fused
reduce-scatter + sharded AdamW kernel. Dense pull of the QKV weights = the all-gather fused into the QKV
GEMM (``ops.gemm.ag_linear``): each layer's ``W_qkv`` is its own table with ``scatter_peers=False``, so
after a push only the owner's rows are current and the first consumer gathers the rest over NVLink while
it already multiplies the local rows. Attention itself is model code, not a parameter-server path: it uses
``torch.nn.functional.scaled_dot_product_attention``; layer norm and GELU are torch ops.

The reference ships no model code (it is a storage service); this is the dense-table consumer.
"""
from __future__ import annotations

import argparse
import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from .._lib import C
from ..ops import gemm as G
from ..ops.dense import DenseTable
from ..ops.sparse import _dist_info, _stream


@dataclass
class GPTConfig:
    n_layer: int = 24
    d_model: int = 2048
    n_head: int = 16
    d_ff: int = 8192
    vocab: int = 50304
    seq_len: int = 2048
    lr: float = 3e-4
    weight_decay: float = 0.1

    def n_params(self) -> int:
        d, f = self.d_model, self.d_ff
        return self.vocab * d + self.seq_len * d + self.n_layer * (3 * d * d + d * d + 2 * d * f + 9 * d + f) + 2 * d


class _PSLinear(torch.autograd.Function):
    """y = x W^T + b on the tcgen05 GEMM; the weight / bias gradients are accumulated into the dense table's
    fp32 gradient views instead of being returned to autograd."""

    @staticmethod
    def forward(ctx, x, w, b, w_grad, b_grad, ag_table, ag_name):
        x2 = x.reshape(-1, x.shape[-1])
        if ag_table is not None:
            y = G.ag_linear(x2, ag_table, ag_name, bias=b)
        else:
            y = G.gemm(x2, w, bias=b)
        ctx.save_for_backward(x2, w)
        ctx.w_grad, ctx.b_grad = w_grad, b_grad
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = G.gemm(dy2, w, b_mn=True)
        G.gemm(dy2, x2, a_mn=True, b_mn=True, out=ctx.w_grad, accumulate=True)
        if ctx.b_grad is not None:
            rc = C.bias_grad(dy2.data_ptr(), dy2.stride(0), dy2.shape[0], dy2.shape[1], ctx.b_grad.data_ptr(), _stream())
            if rc != 0:
                raise RuntimeError(f"bias_grad failed: {rc}")
        return dx.view(ctx.shape), None, None, None, None, None, None


class GPT:
    def __init__(self, cfg: GPTConfig, *, device=None, group=None, seed: int = 0, fuse_qkv_gather: bool = True):
        self.cfg = cfg
        self.group = group
        self.world, self.rank = _dist_info(group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        d, f, L = cfg.d_model, cfg.d_ff, cfg.n_layer
        opt = dict(lr=cfg.lr, weight_decay=cfg.weight_decay, beta2=0.95)
        shapes: Dict[str, tuple] = {"wte": (cfg.vocab, d), "wpe": (cfg.seq_len, d), "lnf.g": (d,), "lnf.b": (d,)}
        for i in range(L):
            shapes.update({f"h{i}.ln1.g": (d,), f"h{i}.ln1.b": (d,), f"h{i}.qkv.b": (3 * d,), f"h{i}.proj.w": (d, d),
                           f"h{i}.proj.b": (d,), f"h{i}.ln2.g": (d,), f"h{i}.ln2.b": (d,), f"h{i}.fc.w": (f, d),
                           f"h{i}.fc.b": (f,), f"h{i}.out.w": (d, f), f"h{i}.out.b": (d,)})
        # the QKV weights can be gathered lazily by their consumer: one table per layer, rows sharded by rank
        self.lazy_qkv = fuse_qkv_gather and self.world > 1 and (3 * d) % (256 * self.world) == 0
        if not self.lazy_qkv:
            for i in range(L):
                shapes[f"h{i}.qkv.w"] = (3 * d, d)
        self.main = DenseTable(shapes, "adamw", opt, grad_dtype=torch.float32, device=self.device, group=group)
        self.qkv: List[Optional[DenseTable]] = []
        for i in range(L):
            self.qkv.append(DenseTable({"w": (3 * d, d)}, "adamw", opt, grad_dtype=torch.float32, device=self.device, group=group,
                                       scatter_peers=False) if self.lazy_qkv else None)
        gen = torch.Generator().manual_seed(seed)
        init = {}
        for name, shape in shapes.items():
            if name.endswith(".g"):
                init[name] = torch.ones(shape)
            elif name.endswith(".b"):
                init[name] = torch.zeros(shape)
            else:
                std = 0.02 / math.sqrt(2 * L) if (".proj.w" in name or ".out.w" in name) else 0.02
                init[name] = torch.randn(shape, generator=gen) * std
        self.main.load(init)
        for i, t in enumerate(self.qkv):
            if t is not None:
                t.load({"w": torch.randn((3 * d, d), generator=gen) * 0.02})
        # small parameters go through autograd as leaves that alias the table; their .grad is folded in later
        self._leaves = {}
        for name in shapes:
            if name in ("wte", "wpe") or ".ln" in name or name.startswith("lnf."):
                self._leaves[name] = self.main.params[name].requires_grad_(True)
        self.tables = [self.main] + [t for t in self.qkv if t is not None]

    # ------------------------------------------------------------------------------------------
    def _linear(self, x, wname, bname, ag_table=None):
        P, Gd = self.main.params, self.main.grads
        if ag_table is not None:
            return _PSLinear.apply(x, ag_table.params["w"], P[bname], ag_table.grads["w"], Gd[bname], ag_table, "w")
        return _PSLinear.apply(x, P[wname], P[bname], Gd[wname], Gd[bname], None, None)

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None):
        cfg = self.cfg
        B, T = tokens.shape
        lv = self._leaves
        x = F.embedding(tokens, lv["wte"]) + lv["wpe"][:T]
        for i in range(cfg.n_layer):
            h = F.layer_norm(x, (cfg.d_model,), lv[f"h{i}.ln1.g"], lv[f"h{i}.ln1.b"])
            qkv = self._linear(h, f"h{i}.qkv.w", f"h{i}.qkv.b", self.qkv[i])
            q, k, v = qkv.view(B, T, 3, cfg.n_head, cfg.d_model // cfg.n_head).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            a = a.transpose(1, 2).reshape(B, T, cfg.d_model)
            x = x + self._linear(a, f"h{i}.proj.w", f"h{i}.proj.b")
            h = F.layer_norm(x, (cfg.d_model,), lv[f"h{i}.ln2.g"], lv[f"h{i}.ln2.b"])
            h = F.gelu(self._linear(h, f"h{i}.fc.w", f"h{i}.fc.b"), approximate="tanh")
            x = x + self._linear(h, f"h{i}.out.w", f"h{i}.out.b")
        x = F.layer_norm(x, (cfg.d_model,), lv["lnf.g"], lv["lnf.b"])
        # tied output embedding: the GEMM's weight gradient and the embedding's gradient both land in wte's slot
        logits = _PSLinear.apply(x, self.main.params["wte"], None, self.main.grads["wte"], None, None, None)
        if targets is None:
            return logits, None
        loss = F.cross_entropy(logits.float().view(-1, cfg.vocab), targets.reshape(-1))
        return logits, loss

    def zero_grads(self) -> None:
        for t in self.tables:
            t.zero_grads()
        for p in self._leaves.values():
            p.grad = None

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor, micro_batches: int = 1) -> torch.Tensor:
        """One optimizer step on this rank's batch (split into ``micro_batches`` accumulation steps): forward,
        backward, then the collective dense push of every table."""
        self.zero_grads()
        total = torch.zeros((), device=self.device)
        for tk, tg in zip(tokens.chunk(micro_batches), targets.chunk(micro_batches)):
            _, loss = self.forward(tk, tg)
            (loss / micro_batches).backward()
            total += loss.detach() / micro_batches
        for name, p in self._leaves.items():
            if p.grad is not None:
                self.main.grads[name].add_(p.grad.float())
        for t in self.tables:
            t.push()
        return total

    def check(self) -> None:
        for t in self.tables:
            t.check()
        G.check_gemm_errors()

    def save_checkpoint(self, uri: str) -> None:
        """Collective, between steps: every dense table (values, optimizer slots, step count) under ``<uri>/table_<i>``."""
        from ..parallel import checkpoint
        torch.cuda.synchronize(self.device)
        for i, t in enumerate(self.tables):
            checkpoint.dump_dense(t, f"{uri.rstrip('/')}/table_{i}")

    def load_checkpoint(self, uri: str) -> None:
        """Collective, between steps; the checkpoint may come from a job with another number of ranks."""
        from ..parallel import checkpoint
        torch.cuda.synchronize(self.device)
        for i, t in enumerate(self.tables):
            checkpoint.load_dense(t, f"{uri.rstrip('/')}/table_{i}")


def _bench(args) -> None:
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = GPTConfig(n_layer=args.layers)
    model = GPT(cfg, fuse_qkv_gather=not args.no_fuse)
    B = args.seqs_per_gpu
    gen = torch.Generator().manual_seed(local)
    tok = torch.randint(0, cfg.vocab, (B, cfg.seq_len + 1), generator=gen).pin_memory()
    d_tok = torch.empty_like(tok, device="cuda")
    for _ in range(args.warmup):
        d_tok.copy_(tok, non_blocking=True)
        model.train_step(d_tok[:, :-1], d_tok[:, 1:], args.micro)
    model.check()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        d_tok.copy_(tok, non_blocking=True)
        loss = model.train_step(d_tok[:, :-1], d_tok[:, 1:], args.micro)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    model.check()
    tokens = B * cfg.seq_len * world
    flops = 6 * cfg.n_params() * tokens + 12 * cfg.n_layer * cfg.d_model * cfg.seq_len * tokens
    if local == 0:
        print(json.dumps({"metric": "gpt_tokens_per_sec", "value": tokens / (ms / 1e3), "n_gpus": world, "ms_per_step": ms,
                          "model_tflops_per_gpu": flops / (ms / 1e3) / 1e12 / world, "layers": cfg.n_layer,
                          "params": cfg.n_params(), "global_batch_seqs": B * world, "seq_len": cfg.seq_len,
                          "qkv_gather_fused": model.lazy_qkv, "loss": float(loss.item())}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="GPT dense-path benchmark (config 4): python -m parameter_server_b200.models.gpt")
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--seqs-per-gpu", type=int, default=8)
    ap.add_argument("--micro", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--no-fuse", action="store_true", help="all-gather the QKV weights in the dense push instead of in the GEMM")
    _bench(ap.parse_args())
