"""SparseTable: the torch-facing sparse parameter table.

One instance per rank (one process per GPU). ``pull`` and ``push`` are collective calls: every
rank of the group calls them in the same order, and the fused kernels exchange keys, rows and
gradients through NVLink peer memory (see ``csrc/kernels/sparse_fused.cu``). They stand for
``PullHandler::pull`` and ``PushHandler::async_push / sync_push / store``
(pico-ps/handler/PullHandler.h:45-99, pico-ps/handler/PushHandler.h:43-107).

On a machine without CUDA the same class runs on the host storage back-end (``HostTable``), which
is also the numerical oracle of the kernels.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .._lib import C
from ..utils.status import StatusError, raise_if_error
from ..utils.trace import nvtx
from .optim import OPTIMIZERS, make_opt_config, set_adam_step


def _dist_info(group=None):
    import torch.distributed as dist

    if group == "none":  # a private single-rank table inside a distributed job
        return 1, 0
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class SparseTable:
    """Sharded ``int64 key -> fp32[dim]`` table with optimizer slots kept next to each row.

    ``pull`` can deliver bfloat16 rows (``supports_bf16_out``): the table stays fp32.

    Args:
        dim: embedding width (a multiple of 4).
        optimizer: ``sgd | adagrad | ftrl | adam | adamw | sum | set``; options go in ``opt_kwargs``.
        capacity: expected number of keys held by THIS rank (sizes the index; the row pool grows).
        max_keys: largest number of key positions in one pull / push call on this rank.
        n_shards: global shard count G (default: world size); keys map to shards with
            ``jump_consistent_hash(murmur(key), G)`` and shards to ranks with ``shard_owner``.
        sync: allocate the per-row delta section needed by ``sync_push`` + ``store``.
        replicate: allocate the replica log, so that pushes can keep a mirror on the next rank exact
            (``parallel.ReplicaSet(table, in_push=True)``).
        read_only: pulls never insert (predictor tables).
        device: ``cuda`` device, or ``cpu`` for the host back-end.
    """

    supports_bf16_out = True

    def __init__(self, dim: int, optimizer: str = "adagrad", opt_kwargs: Optional[dict] = None, *,
                 capacity: int = 1 << 20, max_keys: int = 1 << 20, n_shards: Optional[int] = None,
                 sync: bool = False, read_only: bool = False, init_range: float = 0.01, seed: int = 0,
                 device=None, group=None, pair_capacity: int = 0, wait_limit_s: float = 10.0,
                 max_rows: int = 0, slab_shift: Optional[int] = None, memory_limit_bytes: int = 0, replicate: bool = False):
        if dim % 4:
            raise ValueError("dim must be a multiple of 4")
        self.dim = dim
        self.group = group
        self.world, self.rank = _dist_info(group)
        self.n_shards = int(n_shards or self.world)
        if self.n_shards < 1:
            raise ValueError("n_shards must be at least 1")
        self.read_only = read_only
        self.sync = bool(sync)
        self.opt = make_opt_config(optimizer, **(opt_kwargs or {}))
        self.opt_name = optimizer.lower()
        self.step = 0
        self.max_keys = int(max_keys)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        self._plan_keys = None
        if self.is_cuda:
            tc = C.GpuTableConfig()
            tc.device = self.device.index if self.device.index is not None else torch.cuda.current_device()
            tc.dim = dim
            tc.opt_type = self.opt.type
            tc.sync_delta = sync
            tc.index_capacity = max(2 * int(capacity), 1024)
            tc.max_rows = int(max_rows)
            stride_bytes = 4 * dim * (1 + C.opt_num_slots(self.opt.type) + (1 if sync else 0))
            if slab_shift is None:
                # slabs of about 256 MB, at least 4096 rows
                slab_shift = max(12, min(22, int(np.log2(max(1, (256 << 20) // stride_bytes)))))
            tc.slab_shift = slab_shift
            tc.init_seed = seed
            tc.init_range = init_range
            tc.slot_init0 = self.opt.slot_init0
            tc.slot_init1 = self.opt.slot_init1
            tc.soft_limit_bytes = int(memory_limit_bytes)
            tc.hard_limit_bytes = int(memory_limit_bytes)
            with torch.cuda.device(self.device):
                self.table = C.GpuTable(tc)
                ec = C.SparseEngineConfig()
                ec.world, ec.rank = self.world, self.rank
                ec.max_keys = self.max_keys
                ec.pair_capacity = int(pair_capacity)
                ec.n_shards = self.n_shards
                ec.wait_limit_s = wait_limit_s
                ec.replicate = bool(replicate)   # room for the replica log (see parallel.ReplicaSet(in_push=True))
                self.engine = C.SparseEngine(self.table, ec)
                if self.world > 1:
                    self._connect()
        else:
            hc = C.HostTableConfig()
            hc.dim = dim
            hc.opt_type = self.opt.type
            hc.sync_delta = sync
            hc.n_shards = self.n_shards
            hc.init_seed = seed
            hc.init_range = init_range
            hc.slot_init0 = self.opt.slot_init0
            hc.slot_init1 = self.opt.slot_init1
            hc.soft_limit_bytes = int(memory_limit_bytes)
            hc.hard_limit_bytes = int(memory_limit_bytes)
            self.table = C.HostTable(hc)
            self.engine = None
            self._shard_owner = [s % self.world for s in range(self.n_shards)]
            for s in range(self.n_shards):
                if self.world == 1 or self._shard_owner[s] == self.rank:
                    self.table.create_shard(s)

    # ------------------------------------------------------------------------------------------
    def _connect(self) -> None:
        import torch.distributed as dist

        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(self.engine.ipc_handle()), group=self.group)
        raise_if_error(self.engine.connect(handles))
        dist.barrier(group=self.group)

    @property
    def shard_owner(self) -> Sequence[int]:
        return list(self.engine.shard_owner()) if self.is_cuda else list(self._shard_owner)

    def set_shard_owner(self, owner: Sequence[int]) -> None:
        if self.is_cuda:
            raise_if_error(self.engine.set_shard_owner(list(owner)))
        else:
            self._shard_owner = list(owner)

    # ------------------------------------------------------------------------------------------
    def pull(self, keys: torch.Tensor, bag_size: int = 1, mean: bool = False, *, insert: Optional[bool] = None,
             out: Optional[torch.Tensor] = None, for_push: bool = True, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Rows (sum/mean pooled over ``bag_size`` consecutive keys) of ``keys``; missing keys are
        inserted with their initial value unless the table is read-only. ``out`` (or ``out_dtype``) may be
        bfloat16: the table stays fp32, the rows are rounded where they are read."""
        insert = (not self.read_only) if insert is None else insert
        keys = keys.reshape(-1)
        n = keys.numel()
        if self.is_cuda:
            if keys.dtype != torch.int64 or not keys.is_cuda:
                raise TypeError("keys must be a CUDA int64 tensor")
            keys = keys.contiguous()
            if out is None:
                out = torch.empty((n // bag_size, self.dim), dtype=out_dtype or torch.float32, device=self.device)
            elif (out.dtype not in (torch.float32, torch.bfloat16) or not out.is_cuda or not out.is_contiguous()
                  or out.numel() != (n // bag_size) * self.dim):
                raise ValueError("out must be a contiguous CUDA float32 or bfloat16 tensor of n / bag_size rows of dim columns")
            flags = C.FUSED_COPY_ROWS
            if out.dtype == torch.bfloat16:
                # the consumer's activation dtype: rows are rounded once, by their owner, and cross NVLink as bf16
                flags |= C.FUSED_OUT_BF16
            if insert:
                flags |= C.FUSED_INSERT
            if for_push:
                flags |= C.FUSED_PREPARE_PUSH
            if mean:
                flags |= C.FUSED_MEAN
            with nvtx("ps.sparse_pull"):
                st = self.engine.pull(keys.data_ptr(), n, bag_size, out.data_ptr(), flags, _stream())
            raise_if_error(st)
            self._plan_keys = keys  # keep the key buffer alive until the push
            return out
        if self.world > 1:
            rows = self._cpu_collective_pull(keys.cpu().numpy(), bag_size, mean, insert)
        else:
            st, rows = self.table.pull(keys.cpu().numpy(), bag_size, mean, insert)
            raise_if_error(st)
        self._plan_keys = (keys.cpu().numpy().copy(), bag_size, mean)
        res = torch.from_numpy(rows)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def plan(self, keys: torch.Tensor, bag_size: int = 1, mean: bool = False) -> None:
        """Prepare a push for ``keys`` without returning rows (push without a preceding pull)."""
        keys = keys.reshape(-1)
        if self.is_cuda:
            if keys.dtype != torch.int64 or not keys.is_cuda:
                raise TypeError("keys must be a CUDA int64 tensor")   # a host pointer must never reach the kernel
            keys = keys.contiguous()
            flags = C.FUSED_INSERT | C.FUSED_PREPARE_PUSH | (C.FUSED_MEAN if mean else 0)
            raise_if_error(self.engine.pull(keys.data_ptr(), keys.numel(), bag_size, 0, flags, _stream()))
            self._plan_keys = keys
        else:
            self._plan_keys = (keys.cpu().numpy().copy(), bag_size, mean)

    def push(self, grads: torch.Tensor, keys: Optional[torch.Tensor] = None, *, sync: bool = False,
             bag_size: int = 1, mean: bool = False) -> None:
        """Apply gradients (w.r.t. the pooled pull output) to the rows of the last pull's keys, or of
        ``keys`` when given. ``sync=True`` buffers into the delta section until :meth:`store`."""
        if keys is not None:
            self.plan(keys, bag_size, mean)
        if self._plan_keys is None:
            raise RuntimeError("push without keys needs a preceding pull")
        self.step += 1
        if self.opt.type == C.OPT_ADAM:
            set_adam_step(self.opt, self.step)
        if self.is_cuda:
            if grads.dtype != torch.float32:
                grads = grads.float()
            grads = grads.contiguous()
            if not grads.is_cuda or grads.numel() % self.dim:
                raise ValueError("grads must be a CUDA tensor with one row of dim columns per pulled bag")
            flags = C.FUSED_SYNC_PUSH if sync else 0
            with nvtx("ps.sparse_push"):
                # the engine refuses a gradient buffer whose row count differs from the plan's bags
                raise_if_error(self.engine.push(grads.data_ptr(), grads.numel() // self.dim, self.opt, flags, _stream()))
            self._last_grads = grads  # keep alive until the kernel ran
        else:
            k, bag, mn = self._plan_keys
            g = grads.detach().cpu().float().numpy().reshape(-1, self.dim)
            if self.world > 1:
                self._cpu_collective_push(k, g, bag, mn, sync)
            else:
                raise_if_error(self.table.push(k, g, self.opt, bag, mn, sync))

    # ---- host back-end with more than one rank: the collective protocol over the process group ---------
    # The same owner-computes scheme as the fused kernels, spelled out with object collectives (any backend,
    # e.g. gloo): every rank dedups its keys, the owner of a key serves every requester in rank order (so
    # inserts and the cross-rank gradient fold happen in one fixed order), rows travel back. It exists for
    # CPU-only jobs and as the multi-process oracle of the host-side logic; it is not a fast path.
    def _owners_of(self, keys_np: np.ndarray) -> np.ndarray:
        return C.sparse_shards_of(np.ascontiguousarray(keys_np, dtype=np.int64), self.n_shards, list(self._shard_owner))

    def _cpu_collective_pull(self, keys_np: np.ndarray, bag_size: int, mean: bool, insert: bool) -> np.ndarray:
        import torch.distributed as dist

        uniq, inv = np.unique(keys_np, return_inverse=True)
        asked = [None] * self.world
        dist.all_gather_object(asked, uniq, group=self.group)
        served = []
        for r in range(self.world):                      # requester order: inserts happen in one fixed order
            ks = asked[r]
            mine = ks[self._owners_of(ks) == self.rank] if len(ks) else ks
            st, rows = self.table.pull(mine.astype(np.int64), 1, False, insert)
            raise_if_error(st)
            served.append(rows)
        answers = [None] * self.world
        dist.all_gather_object(answers, served, group=self.group)
        owners = self._owners_of(uniq)
        rows = np.empty((len(uniq), self.dim), dtype=np.float32)
        for o in range(self.world):
            rows[owners == o] = answers[o][self.rank]
        out = rows[inv]
        if bag_size > 1:
            out = out.reshape(-1, bag_size, self.dim).sum(axis=1, dtype=np.float32)
            if mean:
                out = (out / np.float32(bag_size)).astype(np.float32)
        return out

    def _cpu_collective_push(self, keys_np: np.ndarray, grads: np.ndarray, bag_size: int, mean: bool, sync: bool) -> None:
        import torch.distributed as dist

        per_pos = np.repeat(grads, bag_size, axis=0) if bag_size > 1 else grads
        if bag_size > 1 and mean:
            per_pos = (per_pos / np.float32(bag_size)).astype(np.float32)
        uniq, inv = np.unique(keys_np, return_inverse=True)
        agg = np.zeros((len(uniq), self.dim), dtype=np.float32)
        np.add.at(agg, inv, per_pos.astype(np.float32))   # client-side pre-aggregation
        sent = [None] * self.world
        dist.all_gather_object(sent, (uniq, agg), group=self.group)
        ks, gs = [], []
        for r in range(self.world):                      # fold the sources in rank order, then ONE update per row
            u, a = sent[r]
            if len(u):
                own = self._owners_of(u) == self.rank
                ks.append(u[own])
                gs.append(a[own])
        if ks and sum(len(k) for k in ks):
            raise_if_error(self.table.push(np.concatenate(ks).astype(np.int64), np.concatenate(gs), self.opt, 1, False, sync))

    def store(self) -> None:
        """Fold the buffered sync pushes into the weights (OP_STORE)."""
        if self.is_cuda:
            raise_if_error(self.table.store_delta(self.opt, _stream()))
        else:
            raise_if_error(self.table.store(self.opt))

    def reserve(self, n_new_rows: int, exact: bool = False) -> None:
        """Make room for ``n_new_rows`` more rows now (grows the slab pool on the host). Needed before
        a pull is captured in, or replayed from, a CUDA graph, where the call itself cannot allocate.
        The default never blocks: it reads counters that the device mirrored to pinned memory and adds a
        3x margin for calls still in flight. ``exact=True`` reads the counters synchronously and
        allocates exactly what is asked (for sizing a table up front)."""
        if self.is_cuda:
            # the index grows with the table (load kept under one half), also between replays of a captured step
            st = self.table.maybe_grow(int(n_new_rows))
            if not st.ok() and st.code() != C.StatusCode.OUT_OF_MEMORY:
                raise_if_error(st)
            st = self.table.reserve_exact(int(n_new_rows)) if exact else self.table.reserve_rows(int(n_new_rows))
            if not st.ok() and st.code() != C.StatusCode.OUT_OF_MEMORY:
                raise_if_error(st)

    def check(self) -> None:
        """Synchronise and raise :class:`StatusError` if a kernel reported an error."""
        if self.is_cuda:
            raise_if_error(self.engine.check(_stream()))

    def status(self):
        return self.engine.check(_stream()) if self.is_cuda else C.Status()

    def reset(self) -> None:
        """Re-arm the engine after a fatal device status (time-out, error). Every rank of the group must call it."""
        if self.is_cuda:
            raise_if_error(self.engine.reset(_stream()))

    def set_deterministic(self, on: bool = True) -> None:
        """Reproducible pushes: duplicate keys are summed in position order and the owners fold the ranks in rank
        order, so the table after a push is a function of the requests alone (slower on batches with very hot keys)."""
        if self.is_cuda:
            raise_if_error(self.engine.set_deterministic(bool(on)))

    def set_grad_wire_bf16(self, on: bool = True) -> None:
        """Ship the merged gradient rows of a push to their owners as bf16 (the sums on both sides stay fp32). Halves
        the bytes of the push's NVLink phase; for models whose gradients come out of bf16 arithmetic anyway."""
        if self.is_cuda:
            self.engine.set_grad_wire_bf16(bool(on))

    def set_sm_budget(self, pull_sms: int = 0, push_sms: int = 0) -> None:
        """Bound the fused pull / push kernels to that many SMs (0 = all). One of their CTAs fills an SM, so the
        remaining SMs stay free, whole, for kernels of another stream that run at the same time."""
        if self.is_cuda:
            self.engine.set_sm_budget(int(pull_sms), int(push_sms))

    # ------------------------------------------------------------------------------------------
    def size(self) -> int:
        return int(self.table.size())

    def memory_usage(self) -> int:
        return int(self.table.memory_usage())

    def storage_info(self, collective: bool = False):
        """What ``Client.query_storage_info`` answers on the service path: one record per local shard,
        ``{"node_id": rank, "shard_id", "item_number", "memory_usage"}`` (the table's bytes spread evenly over its
        shards, as there); with ``collective`` the records of all ranks."""
        mine = [s for s in range(self.n_shards) if self.world == 1 or self.shard_owner[s] == self.rank]
        if self.is_cuda:
            st, counts = self.table.shard_counts(self.n_shards, _stream())
            raise_if_error(st)
            items = {s: int(counts[s]) for s in mine}
        else:
            items = {s: int(self.table.shard_size(s)) for s in mine}
        per = self.memory_usage() // max(1, len(mine))
        info = [{"node_id": self.rank, "shard_id": s, "item_number": items[s], "memory_usage": per} for s in mine]
        if collective and self.world > 1:
            import torch.distributed as dist
            parts = [None] * self.world
            dist.all_gather_object(parts, info, group=self.group)
            info = [r for p in parts for r in p]
        return info

    def get_rows(self, keys: torch.Tensor, emb_only: bool = True):
        """Read rows of LOCAL keys without inserting. Returns (rows, found)."""
        keys = keys.reshape(-1)
        if self.is_cuda:
            if keys.dtype != torch.int64 or not keys.is_cuda:
                raise TypeError("keys must be a CUDA int64 tensor")
            keys = keys.contiguous()
            w = self.dim if emb_only else self.table.stride()
            out = torch.empty((keys.numel(), w), dtype=torch.float32, device=self.device)
            found = torch.empty(keys.numel(), dtype=torch.int32, device=self.device)
            raise_if_error(self.table.get_rows(keys.data_ptr(), keys.numel(), out.data_ptr(), found.data_ptr(),
                                               emb_only, _stream()))
            return out, found
        rows, found = self.table.get_rows(keys.cpu().numpy(), emb_only)
        return torch.from_numpy(rows), torch.from_numpy(found)

    def set_rows(self, keys: torch.Tensor, rows: torch.Tensor, emb_only: bool = False) -> None:
        """Insert / overwrite rows of LOCAL keys (DirectPush)."""
        keys = keys.reshape(-1)
        if self.is_cuda:
            keys = keys.contiguous()
            rows = rows.contiguous().float()
            width = self.dim if emb_only else self.table.stride()
            if not keys.is_cuda or not rows.is_cuda or keys.dtype != torch.int64 or rows.numel() != keys.numel() * width:
                raise ValueError("set_rows needs CUDA int64 keys and one row of %d floats per key" % width)
            raise_if_error(self.table.set_rows(keys.data_ptr(), rows.data_ptr(), keys.numel(), emb_only, _stream()))
        else:
            raise_if_error(self.table.set_rows(keys.cpu().numpy(), rows.cpu().float().numpy(), emb_only))

    def erase_keys(self, keys: torch.Tensor) -> int:
        keys = keys.reshape(-1)
        if self.is_cuda:
            if keys.dtype != torch.int64 or not keys.is_cuda:
                raise TypeError("keys must be a CUDA int64 tensor")
            keys = keys.contiguous()
            st, n = self.table.erase_keys(keys.data_ptr(), keys.numel(), _stream())
            raise_if_error(st)
            return int(n)
        return int(self.table.erase_keys(keys.cpu().numpy()))

    def export(self, shard: int = -1, batch: int = 1 << 18, dirty_only: bool = False):
        """Iterate ``(keys, rows)`` batches of the local entries (of one shard when ``shard >= 0``).
        ``rows`` carries the full row: embedding, optimizer slots and, if present, the sync delta."""
        if self.is_cuda:
            stride = self.table.stride()
            cap = self.table.index_capacity()
            window = min(cap, max(1024, batch))
            kbuf = torch.empty(window, dtype=torch.int64, device=self.device)
            rbuf = torch.empty((window, stride), dtype=torch.float32, device=self.device)
            cursor = 0
            mode = 4 if dirty_only else (1 if shard >= 0 else 0)
            while cursor < cap:
                st, n, cursor = self.table.export_window(cursor, window, mode, shard, self.rank, self.n_shards, 0,
                                                         kbuf.data_ptr(), rbuf.data_ptr(), _stream())
                raise_if_error(st)
                if n:
                    k, r = kbuf[:n].clone(), rbuf[:n].clone()
                    if dirty_only and shard >= 0:
                        sel = torch.from_numpy(C.sparse_shards_of(k.cpu().numpy(), self.n_shards) == shard).to(self.device)
                        k, r = k[sel], r[sel]
                    if k.numel():
                        yield k, r
        else:
            shards = [shard] if shard >= 0 else self.table.shard_list()
            for s in shards:
                cursor, finished = 0, False
                while not finished:
                    k, r, cursor, finished = self.table.export_shard(s, cursor, batch, dirty_only)
                    if len(k):
                        yield torch.from_numpy(k), torch.from_numpy(r)

    # ---- scans over the local entries: the for_each / erase_if verbs of the operator API ------------
    # A scan is written with torch over batches of (keys, rows) that lie where the table lies (device tensors for
    # a CUDA table: nothing crosses PCIe). Every rank scans its own entries; ``collective=True`` combines the
    # answers of all ranks. Parity: pico-ps/operator/ForEachOperator.h:150-233 (reading scan, init / for_each /
    # merge), :277-359 (writing scan), pico-ps/operator/EraseIfOperator.h:17-58.
    def _predicate(self, spec):
        """A built-in predicate ``{"type": "key_mod", "mod": m, "rem": r} | {"type": "l2_below", "threshold": t} |
        {"type": "slot0_below", "threshold": t} | {"type": "all"}`` (the menu of the RPC path's EraseIfOperator) as
        a function of a batch."""
        if callable(spec):
            return spec
        kind, dim = spec.get("type"), self.dim
        if kind == "key_mod":
            mod, rem = int(spec.get("mod", 2)), int(spec.get("rem", 1))
            return lambda k, r: torch.remainder(k, mod) == rem
        if kind == "l2_below":
            t = float(spec.get("threshold", 0.0))
            return lambda k, r: r[:, :dim].double().pow(2).sum(1).sqrt() < t
        if kind == "slot0_below":
            if self.table.stride() < 2 * dim:
                raise ValueError("slot0_below needs an optimizer with a slot")
            t = float(spec.get("threshold", 0.0))
            return lambda k, r: r[:, dim:2 * dim].double().mean(1) < t
        if kind == "all":
            return lambda k, r: torch.ones(k.numel(), dtype=torch.bool, device=k.device)
        raise ValueError("unknown predicate %r" % (kind,))

    def _all_reduce(self, value: torch.Tensor, op: str) -> torch.Tensor:
        if self.world > 1:
            import torch.distributed as dist
            value = value.to(self.device if self.is_cuda else "cpu")
            dist.all_reduce(value, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM, group=self.group)
        return value

    def erase_if(self, predicate, *, collective: bool = False, batch: int = 1 << 18) -> int:
        """Erase the local entries for which ``predicate(keys, rows) -> bool mask`` holds (or a built-in predicate
        given as a dict, see ``_predicate``). Returns the number erased here, or on all ranks with ``collective``."""
        pred = self._predicate(predicate)
        doomed = []
        for k, r in self.export(batch=batch):
            m = pred(k, r)
            if bool(m.any()):
                doomed.append(k[m])
        # erased after the walk: an erase may make a host index rebuild itself, which would move the entries under it
        n = self.erase_keys(torch.cat(doomed)) if doomed else 0
        if collective:
            n = int(self._all_reduce(torch.tensor([n], dtype=torch.int64), "sum").item())
        return n

    def for_each(self, fn=None, *, section: int = 0, collective: bool = False, batch: int = 1 << 18):
        """Reading scan. With ``fn(keys, rows)``: called per batch, the list of its results is returned (the caller
        merges). Without: the built-in statistics of row section ``section`` (0 = embedding, 1 / 2 = optimizer
        slots) as ``{"count", "sum", "sum_sq", "max_abs"}``, over all ranks with ``collective``."""
        if fn is not None:
            return [fn(k, r) for k, r in self.export(batch=batch)]
        dim = self.dim
        if (section + 1) * dim > self.table.stride():
            raise ValueError("no such row section")
        acc = torch.zeros(3, dtype=torch.float64)
        mx = torch.zeros(1, dtype=torch.float64)
        for k, r in self.export(batch=batch):
            v = r[:, section * dim:(section + 1) * dim].double()
            acc += torch.stack([torch.tensor(float(k.numel()), dtype=torch.float64, device=v.device), v.sum(), v.pow(2).sum()]).cpu()
            mx = torch.maximum(mx, v.abs().max().reshape(1).cpu())
        if collective:
            acc, mx = self._all_reduce(acc, "sum").cpu(), self._all_reduce(mx, "max").cpu()
        return {"count": int(acc[0].item()), "sum": acc[1].item(), "sum_sq": acc[2].item(), "max_abs": mx.item()}

    def for_each_write(self, fn, *, collective: bool = False, batch: int = 1 << 18) -> int:
        """Writing scan: ``fn(keys, rows)`` returns the new rows of the batch (same shape: embedding, optimizer
        slots and, if present, the sync delta) or ``None``; rows that differ are written back. Returns how many
        rows changed here, or on all ranks with ``collective``. Call it between steps: a push that lands between
        the read of a batch and its write-back would be overwritten."""
        n = 0
        for k, r in self.export(batch=batch):
            new = fn(k, r)
            if new is None:
                continue
            if new.shape != r.shape:
                raise ValueError("for_each_write: fn must return rows of the shape it was given")
            new = new.to(dtype=torch.float32)
            changed = (new != r).any(1)
            c = int(changed.sum().item())
            if c:
                self.set_rows(k[changed], new[changed], emb_only=False)   # existing keys: the index does not move
                n += c
        if collective:
            n = int(self._all_reduce(torch.tensor([n], dtype=torch.int64), "sum").item())
        return n

    # ---- cold tier (pinned host DRAM under the HBM table) ---------------------------------------
    def enable_cold_tier(self, capacity_rows: int, window: int = 1 << 16) -> None:
        """Attach a pinned-host tier of ``capacity_rows`` rows (the role of the reference's PMEM tier)."""
        if not self.is_cuda:
            raise RuntimeError("the cold tier sits under a GPU table")
        self.cold = C.HostColdTier(self.table, int(capacity_rows), int(window))

    def spill_cold(self, section: int = 1, threshold: float = 0.0) -> int:
        """Move rows whose mean over row section ``section`` is below ``threshold`` to the cold tier."""
        torch.cuda.current_stream().synchronize()
        st, n = self.cold.spill_if(section, threshold)
        raise_if_error(st)
        return int(n)

    def spill_keys(self, keys: torch.Tensor) -> int:
        k = keys.reshape(-1).cpu().to(torch.int64).contiguous()
        torch.cuda.current_stream().synchronize()
        st, n = self.cold.spill_keys(k.data_ptr(), k.numel())
        raise_if_error(st)
        return int(n)

    def prefetch_cold(self, keys: torch.Tensor) -> int:
        """Bring the rows of ``keys`` (a host tensor, e.g. the next batch while it is still in pinned
        memory) back from the cold tier before they are pulled. Returns how many came back."""
        k = keys.reshape(-1).cpu().to(torch.int64).contiguous()
        st, n = self.cold.fetch(k.data_ptr(), k.numel())
        raise_if_error(st)
        return int(n)

    def prefetch_cold_async(self, keys: torch.Tensor) -> None:
        """Start bringing back the cold rows among ``keys`` (at most one staging window of them) without
        blocking: lookup, packing and the host-to-device copy run on a worker thread and a side stream while
        the current step computes. ``commit_prefetch()`` inserts them."""
        k = keys.reshape(-1).cpu().to(torch.int64).contiguous()
        self.cold.stage_fetch_async(k.data_ptr(), k.numel())

    def commit_prefetch(self) -> int:
        """Insert the rows staged by ``prefetch_cold_async`` (call between two steps, before the pull that
        needs them). Returns how many rows came back."""
        st, n = self.cold.commit_fetch(_stream())
        raise_if_error(st)
        return int(n)

    def clear(self) -> None:
        if self.is_cuda:
            raise_if_error(self.table.clear(_stream()))
        else:
            self.table.clear()

    # ------------------------------------------------------------------------------------------
    def lookup(self, keys: torch.Tensor, bag_size: int = 1, mean: bool = False) -> torch.Tensor:
        """Differentiable pull: the backward pass pushes the gradient to the parameter server."""
        return sparse_lookup(self, keys, bag_size, mean)


class _SparseLookup(torch.autograd.Function):
    """Pull in forward, push in backward (the worker side of a PS training step)."""

    @staticmethod
    def forward(ctx, table: SparseTable, keys: torch.Tensor, bag_size: int, mean: bool, anchor: torch.Tensor):
        ctx.table = table
        return table.pull(keys, bag_size, mean)

    @staticmethod
    def backward(ctx, grad_out):
        ctx.table.push(grad_out)
        return None, None, None, None, None


def sparse_lookup(table: SparseTable, keys: torch.Tensor, bag_size: int = 1, mean: bool = False) -> torch.Tensor:
    # the anchor makes autograd record the node although no input tensor requires grad
    anchor = torch.zeros((), device=table.device if table.is_cuda else "cpu", requires_grad=True)
    return _SparseLookup.apply(table, keys, bag_size, mean, anchor)
