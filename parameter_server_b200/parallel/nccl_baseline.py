"""NCCL-only implementations of the collective sparse and dense paths: the baseline the fused
kernels are measured against (not the product).

Sparse pull = ``torch.unique`` -> sort by owner -> ``all_to_all_single`` (counts, keys) -> local lookup ->
``all_to_all_single`` (rows) -> un-sort / un-dedup. Sparse push = ``index_add_`` of duplicate keys ->
``all_to_all_single`` (keys, gradient rows) -> local optimizer step. Dense push = ``reduce_scatter_tensor``
-> AdamW on the fp32 slice with torch ops -> ``all_gather_into_tensor`` of the bf16 values. The local table
is the same ``GpuTable`` (driven through a private single-rank engine), so the comparison isolates what
the fusion of transport and compute buys. Keys are partitioned with ``key mod world``.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
import torch.distributed as dist

from .._lib import C
from ..ops.optim import make_opt_config
from ..ops.sparse import SparseTable, _dist_info


class NcclSparseTable:
    def __init__(self, dim: int, optimizer: str = "adagrad", opt_kwargs: Optional[dict] = None, *, capacity: int = 1 << 20,
                 max_keys: int = 1 << 20, device=None, group=None, seed: int = 0, **_):
        self.dim = dim
        self.group = group
        self.world, self.rank = _dist_info(group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.is_cuda = True
        # every rank may receive up to world * max_keys keys in the worst case; size for 2x the fair share
        self.local = SparseTable(dim, optimizer, opt_kwargs, capacity=capacity, max_keys=max(max_keys * 2, 1024),
                                 n_shards=1, device=self.device, group="none", seed=seed)
        self.opt = self.local.opt
        self._plan = None

    def _exchange_counts(self, send_counts: torch.Tensor):
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        return send_counts.tolist(), recv_counts.tolist()   # host sync: the split sizes must be known

    def pull(self, keys: torch.Tensor, bag_size: int = 1, mean: bool = False, *, out: Optional[torch.Tensor] = None,
             insert: Optional[bool] = None, for_push: bool = True) -> torch.Tensor:
        keys = keys.reshape(-1)
        uniq, inv = torch.unique(keys, return_inverse=True)
        if self.world == 1:
            rows = self.local.pull(uniq, insert=insert, for_push=False)
            self._plan = (uniq, inv, None, None, None, None)
        else:
            owner = torch.remainder(uniq, self.world)
            order = torch.argsort(owner, stable=True)
            send_keys = uniq[order]
            send_counts = torch.bincount(owner, minlength=self.world)
            sc, rc = self._exchange_counts(send_counts)
            recv_keys = torch.empty(sum(rc), dtype=torch.int64, device=self.device)
            dist.all_to_all_single(recv_keys, send_keys, rc, sc, group=self.group)
            local_rows = self.local.pull(recv_keys, insert=insert, for_push=False) if recv_keys.numel() else \
                torch.empty((0, self.dim), device=self.device)
            back = torch.empty((send_keys.numel(), self.dim), dtype=torch.float32, device=self.device)
            dist.all_to_all_single(back, local_rows, sc, rc, group=self.group)
            rows = torch.empty_like(back)
            rows[order] = back
            self._plan = (uniq, inv, order, sc, rc, recv_keys)
        res = rows[inv]
        if bag_size > 1:
            res = res.view(-1, bag_size, self.dim).sum(1)
            if mean:
                res = res / bag_size
        if out is not None:
            out.copy_(res)
            return out
        return res

    def push(self, grads: torch.Tensor, keys: Optional[torch.Tensor] = None, **_) -> None:
        if keys is not None:
            raise NotImplementedError("baseline push reuses the keys of the last pull")
        uniq, inv, order, sc, rc, recv_keys = self._plan
        agg = torch.zeros((uniq.numel(), self.dim), dtype=torch.float32, device=self.device)
        agg.index_add_(0, inv, grads.reshape(-1, self.dim))
        if self.world == 1:
            self.local.push(agg, keys=uniq)
            return
        send = agg[order]
        recv = torch.empty((sum(rc), self.dim), dtype=torch.float32, device=self.device)
        dist.all_to_all_single(recv, send, rc, sc, group=self.group)
        if recv_keys.numel():
            self.local.push(recv, keys=recv_keys)   # the local engine merges keys that several ranks sent

    def reserve(self, n: int, exact: bool = False) -> None:
        self.local.reserve(n, exact)

    def check(self) -> None:
        self.local.check()

    def size(self) -> int:
        return self.local.size()


class NcclDenseTable:
    """Same interface as :class:`DenseTable`, built from NCCL collectives and torch optimizer math."""

    def __init__(self, shapes: Dict[str, Sequence[int]], optimizer: str = "adamw", opt_kwargs: Optional[dict] = None, *,
                 grad_dtype: torch.dtype = torch.float32, device=None, group=None, **_):
        self.group = group
        self.world, self.rank = _dist_info(group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.opt = make_opt_config(optimizer, **(opt_kwargs or {}))
        self.offsets, off = {}, 0
        for name, shape in shapes.items():
            n = 1
            for s in shape:
                n *= int(s)
            self.offsets[name] = (off, tuple(int(s) for s in shape))
            off += (n + 63) // 64 * 64
        q = 8 * self.world
        self.numel = (max(off, 64) + q - 1) // q * q
        self.shard_len = self.numel // self.world
        self.flat_params = torch.zeros(self.numel, dtype=torch.bfloat16, device=self.device)
        self.flat_grads = torch.zeros(self.numel, dtype=grad_dtype, device=self.device)
        self.master = torch.zeros(self.shard_len, dtype=torch.float32, device=self.device)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.step_count = 0
        self.params = {n: self._slice(self.flat_params, n) for n in self.offsets}
        self.grads = {n: self._slice(self.flat_grads, n) for n in self.offsets}

    def _slice(self, flat, name):
        off, shape = self.offsets[name]
        n = 1
        for s in shape:
            n *= s
        return flat[off:off + n].view(shape)

    def load(self, values: Dict[str, torch.Tensor]) -> None:
        full = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        for name, v in values.items():
            off, _ = self.offsets[name]
            full[off:off + v.numel()] = v.reshape(-1).to(self.device, torch.float32)
        self.flat_params.copy_(full)
        self.master.copy_(full[self.rank * self.shard_len:(self.rank + 1) * self.shard_len])

    def zero_grads(self) -> None:
        self.flat_grads.zero_()

    def pull(self, name: str) -> torch.Tensor:
        return self.params[name]

    def push(self, grad_scale: Optional[float] = None) -> None:
        self.step_count += 1
        o = self.opt
        scale = (1.0 / self.world) if grad_scale is None else grad_scale
        if self.world > 1:
            g = torch.empty(self.shard_len, dtype=self.flat_grads.dtype, device=self.device)
            dist.reduce_scatter_tensor(g, self.flat_grads, group=self.group)
        else:
            g = self.flat_grads
        g = g.float() * scale
        if o.type == C.OPT_ADAM:
            self.m.mul_(o.beta1).add_(g, alpha=1 - o.beta1)
            self.v.mul_(o.beta2).addcmul_(g, g, value=1 - o.beta2)
            if o.weight_decay:
                self.master.mul_(1 - o.lr * o.weight_decay)
            bc1, bc2 = 1 - o.beta1 ** self.step_count, 1 - o.beta2 ** self.step_count
            self.master.addcdiv_(self.m / bc1, (self.v / bc2).sqrt_().add_(o.eps), value=-o.lr)
        else:
            self.master.add_(g, alpha=-o.lr)
        shard = self.master.bfloat16()
        if self.world > 1:
            dist.all_gather_into_tensor(self.flat_params, shard, group=self.group)
        else:
            self.flat_params.copy_(shard)

    def check(self) -> None:
        pass
