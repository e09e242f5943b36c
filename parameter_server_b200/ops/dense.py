"""DenseTable: dense parameters kept on the parameter server.

A table is a set of named tensors packed into one flat buffer; slice ``r`` (the ``r``-th contiguous
``1/world``) is owned by rank ``r``: it keeps the fp32 master weights and optimizer moments of that
slice. ``push()`` is the fused reduce-scatter + optimizer + all-gather kernel
(``csrc/kernels/dense_fused.cu``); after it every rank's bf16 parameter buffer holds the new values, so
``pull(name)`` is a view. Parity: DenseTablePush/PullOperator with a contiguous
``DenseValuePartitioner`` (pico-ps/common/dense_common.h:135-171,
pico-ps/operator/DensePushOperator.h:59-126, pico-ps/operator/DensePullOperator.h:49-116).

Without CUDA the same interface runs on torch CPU tensors (all-reduce over gloo when a process group
exists), which is what the CPU tests exercise.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from .._lib import C
from ..utils.status import raise_if_error
from .optim import make_opt_config, set_adam_step
from ..utils.trace import nvtx
from .sparse import _dist_info, _stream


class _RawCudaBuffer:
    """Zero-copy torch view over device memory owned by the native library."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }
        self._owner = owner


def _view(ptr: int, numel: int, dtype: torch.dtype, device, owner) -> torch.Tensor:
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    raw = torch.as_tensor(_RawCudaBuffer(ptr, nbytes, owner), device=device)
    t = raw.view(dtype)
    t._psb_owner = owner  # keep the native buffer alive as long as the view
    return t


class DenseTable:
    def __init__(self, shapes: Dict[str, Sequence[int]], optimizer: str = "adamw", opt_kwargs: Optional[dict] = None, *,
                 grad_dtype: torch.dtype = torch.float32, device=None, group=None, wait_limit_s: float = 10.0,
                 scatter_peers: bool = True):
        self.group = group
        self.world, self.rank = _dist_info(group)
        self.opt = make_opt_config(optimizer, **(opt_kwargs or {}))
        self.step_count = 0
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        self.grad_dtype = grad_dtype
        # layout: every tensor starts on a 64-element boundary (128 B for bf16: TMA / vector alignment)
        self.offsets: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
        off = 0
        for name, shape in shapes.items():
            shape = tuple(int(s) for s in shape)
            n = 1
            for s in shape:
                n *= s
            self.offsets[name] = (off, shape)
            off += (n + 63) // 64 * 64
        self.numel_used = off
        if self.is_cuda:
            idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
            self.engine = C.DenseEngine(idx, self.world, self.rank, max(off, 64), grad_dtype == torch.bfloat16,
                                        self.opt.type, wait_limit_s)
            self.numel = self.engine.numel()
            # scatter_peers=False: a push leaves the peers' copies stale; the consumer gathers (ops.gemm.ag_linear)
            self.engine.set_scatter_peers(bool(scatter_peers))
            self.scatter_peers = bool(scatter_peers)
            self._ag_ready = None
            self._ag_epoch = 0
            if self.world > 1:
                import torch.distributed as dist
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(self.engine.ipc_handle()), group=group)
                raise_if_error(self.engine.connect(handles))
                dist.barrier(group=group)
            self.flat_params = _view(self.engine.params_ptr(), self.numel, torch.bfloat16, self.device, self.engine)
            self.flat_grads = _view(self.engine.grads_ptr(), self.numel, grad_dtype, self.device, self.engine)
            self.master = _view(self.engine.master_ptr(), self.engine.shard_len(), torch.float32, self.device, self.engine)
        else:
            self.engine = None
            self.numel = max(off, 64)
            self.flat_master = torch.zeros(self.numel, dtype=torch.float32)
            self.flat_params = self.flat_master  # CPU: parameters are the fp32 master itself
            self.flat_grads = torch.zeros(self.numel, dtype=torch.float32)
            self._m = torch.zeros(self.numel) if C.opt_num_slots(self.opt.type) > 0 else None
            self._v = torch.zeros(self.numel) if C.opt_num_slots(self.opt.type) > 1 else None
            if self._m is not None:
                self._m.fill_(self.opt.slot_init0)
        self.params = {n: self._slice(self.flat_params, n) for n in self.offsets}
        self.grads = {n: self._slice(self.flat_grads, n) for n in self.offsets}

    def _slice(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        off, shape = self.offsets[name]
        n = 1
        for s in shape:
            n *= s
        return flat[off:off + n].view(shape)

    # ------------------------------------------------------------------------------------------
    def load(self, values: Dict[str, torch.Tensor]) -> None:
        """Set the parameters from full fp32 tensors (identical on every rank). Tensors that are not named become
        zero: a load replaces the whole table."""
        full = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        for name, v in values.items():
            if name not in self.offsets:
                raise KeyError("no dense tensor %r in this table" % (name,))
            off, shape = self.offsets[name]
            want = 1
            for d in shape:
                want *= int(d)
            if v.numel() != want:
                raise ValueError("dense tensor %r has %d elements, the table holds %s" % (name, v.numel(), tuple(shape)))
            full[off:off + v.numel()] = v.reshape(-1).to(self.device, torch.float32)
        if self.is_cuda:
            raise_if_error(self.engine.load_full(full.data_ptr(), _stream()))
            torch.cuda.current_stream().synchronize()
        else:
            self.flat_master.copy_(full)

    def pull(self, name: str) -> torch.Tensor:
        """The current value of one dense tensor (bf16 view on CUDA, fp32 on CPU)."""
        return self.params[name]

    def zero_grads(self) -> None:
        self.flat_grads.zero_()

    def set_sm_budget(self, sms: int = 0) -> None:
        """Bound the fused dense push to ``sms`` SMs (0 = all): it then runs as CTAs that fill an SM each, so that a
        kernel of another stream (the sparse push of the same step) keeps the other SMs, whichever starts first."""
        if self.is_cuda:
            self.engine.set_sm_budget(int(sms))

    def push(self, grad_scale: Optional[float] = None) -> None:
        """Collective dense push: gradients of all ranks are summed (times ``grad_scale``, default
        ``1/world``), the owner of each slice applies the update rule, new values reach every rank."""
        self.step_count += 1
        if self.opt.type == C.OPT_ADAM:
            set_adam_step(self.opt, self.step_count)
        scale = (1.0 / self.world) if grad_scale is None else grad_scale
        if self.is_cuda:
            with nvtx("ps.dense_push"):
                raise_if_error(self.engine.step(self.opt, scale, _stream()))
            return
        g = self.flat_grads
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(g, group=self.group)
        g = g * scale
        w, o = self.flat_master, self.opt
        if o.type == C.OPT_SGD:
            if o.weight_decay:
                w.mul_(1 - o.lr * o.weight_decay)
            w.add_(g, alpha=-o.lr)
        elif o.type == C.OPT_ADAM:
            self._m.mul_(o.beta1).add_(g, alpha=1 - o.beta1)
            self._v.mul_(o.beta2).addcmul_(g, g, value=1 - o.beta2)
            if o.weight_decay:
                w.mul_(1 - o.lr * o.weight_decay)
            w.addcdiv_(self._m / o.bias_corr1, (self._v / o.bias_corr2).sqrt_().add_(o.eps), value=-o.lr)
        elif o.type == C.OPT_ADAGRAD:
            self._m.addcmul_(g, g)
            w.addcdiv_(g, self._m.sqrt().add_(o.eps), value=-o.lr)
        elif o.type == C.OPT_SUM:
            w.add_(g)
        else:
            raise NotImplementedError("dense tables support sgd / adam(w) / adagrad / sum on the CPU path")

    def check(self) -> None:
        if self.is_cuda:
            raise_if_error(self.engine.check(_stream()))

    def master_slice(self) -> torch.Tensor:
        """fp32 master weights of the slice this rank owns."""
        if self.is_cuda:
            return self.master
        lo = self.numel // self.world * self.rank
        return self.flat_master[lo:lo + self.numel // self.world]
