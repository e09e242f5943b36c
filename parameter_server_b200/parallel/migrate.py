"""Shard migration, replica sync and restore for the collective (GPU) path: rows travel GPU to GPU as
NVLink peer copies into a symmetric inbox, the destination inserts them with the DirectPush kernel.

* :func:`reshard` - change the shard -> rank placement of a :class:`SparseTable` (load balancing, scaling
  the set of serving ranks): every rank exports the rows that no longer belong to it, copies them into the
  new owners' inboxes, inserts what it received and purges what left. The GPU counterpart of the reshard
  transaction (pico-ps/handler/UpdateContextHandler.cpp:62-153, shuffle =
  pico-ps/operator/UpdateContextOperator.h:215-304, purge = :143-193).
* :class:`ReplicaSet` - a second table per rank that mirrors the shards of a partner rank (2x replication).
  ``sync()`` ships only the rows that changed since the last sync (dirty bits), ``restore()`` refills a
  rank's primary table from its mirror on the partner: the GPU counterpart of pushing to every replica
  and of coordinated restore (pico-ps/operator/RestoreOperator.h:94-151,
  pico-ps/service/coordinated_restore/CoordinatedRestoreWorker.cpp:30-46).

All calls are collective over the table's process group; control information (counts) goes through
``torch.distributed``, row data through peer memory.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .._lib import C
from ..ops.dense import _view
from ..ops.sparse import SparseTable
from ..utils.status import raise_if_error
from . import migrate_host as _host


class PeerInbox:
    """Symmetric buffer with one region per source rank; ``send`` is a peer copy into the destination's
    region, ``counts`` are exchanged on the host side."""

    def __init__(self, table: SparseTable, rows_per_pair: int):
        self.table = table
        self.world, self.rank = table.world, table.rank
        self.stride = table.table.stride()
        self.cap = int(rows_per_pair)
        self.rec_bytes = 8 + 4 * self.stride
        dev = table.device.index if table.device.index is not None else torch.cuda.current_device()
        self.buf = C.SymmetricBuffer(dev, self.world * self.cap * self.rec_bytes)
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(self.buf.ipc_handle()), group=table.group)
            raise_if_error(self.buf.connect(handles, self.rank))
            dist.barrier(group=table.group)

    def _region(self, owner_rank: int, src_rank: int):
        base = (self.buf.peer(owner_rank) if self.world > 1 else self.buf.local()) + src_rank * self.cap * self.rec_bytes
        keys = _view(base, self.cap, torch.int64, self.table.device, self.buf)
        rows = _view(base + self.cap * 8, self.cap * self.stride, torch.float32, self.table.device, self.buf).view(self.cap, self.stride)
        return keys, rows

    def region_ptrs(self, owner_rank: int, src_rank: int):
        """Raw device addresses (keys, rows) of the region of ``owner_rank``'s inbox that ``src_rank`` fills."""
        base = (self.buf.peer(owner_rank) if self.world > 1 else self.buf.local()) + src_rank * self.cap * self.rec_bytes
        return base, base + self.cap * 8

    def keys_view(self, owner_rank: int, src_rank: int) -> torch.Tensor:
        return self._region(owner_rank, src_rank)[0]

    def send(self, dst: int, keys: torch.Tensor, rows: torch.Tensor) -> None:
        n = keys.numel()
        if n > self.cap:
            raise ValueError("inbox region too small for this batch")
        k, r = self._region(dst, self.rank)
        k[:n].copy_(keys)          # peer copy over NVLink (plain device-to-device when dst is this rank)
        r[:n].copy_(rows)

    def received(self, src: int, n: int):
        k, r = self._region(self.rank, src)
        return k[:n], r[:n]


def _exchange_counts(table: SparseTable, send_counts: List[int]) -> List[int]:
    if table.world == 1:
        return list(send_counts)
    t = torch.tensor(send_counts, dtype=torch.int64, device=table.device)
    out = torch.empty_like(t)
    dist.all_to_all_single(out, t, group=table.group)
    return out.tolist()


def _ship(table: SparseTable, inbox: PeerInbox, keys: torch.Tensor, rows: torch.Tensor, dest: torch.Tensor,
          target: Optional[SparseTable] = None) -> int:
    """Send (keys, rows) to the ranks in ``dest`` and insert what this rank receives into ``target``."""
    target = target or table
    world = table.world
    if not table.is_cuda:
        return _host.ship(table, keys, rows, dest, target)
    order = torch.argsort(dest, stable=True)
    keys, rows, dest = keys[order], rows[order], dest[order]
    counts = torch.bincount(dest, minlength=world).tolist()
    recv = _exchange_counts(table, counts)
    off = 0
    for r in range(world):
        if counts[r]:
            inbox.send(r, keys[off:off + counts[r]], rows[off:off + counts[r]])
        off += counts[r]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(group=table.group)        # every peer copy has landed
    total = 0
    for src in range(world):
        if recv[src]:
            k, r = inbox.received(src, recv[src])
            target.set_rows(k, r, emb_only=False)
            total += recv[src]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(group=table.group)        # inboxes may be overwritten again
    return total


def route(table: SparseTable, keys: torch.Tensor, owner_dev: Optional[torch.Tensor]) -> torch.Tensor:
    """Shard of every key (``owner_dev`` None) or the rank that owns it under the map ``owner_dev``."""
    if not table.is_cuda:
        return _host.shards_of(table, keys, None if owner_dev is None else owner_dev.tolist()).to(torch.int32)
    out = torch.empty(keys.numel(), dtype=torch.int32, device=table.device)
    rc = C.shard_of_keys(keys.data_ptr(), keys.numel(), table.n_shards, 0 if owner_dev is None else owner_dev.data_ptr(),
                         out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"shard_of_keys failed: {rc}")
    return out


def _any_rank(table: SparseTable, flag: bool) -> bool:
    if table.world == 1:
        return flag
    t = torch.tensor([1 if flag else 0], device=table.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=table.group)
    return bool(t.item())


def stream_to_owners(table: SparseTable, batches, owner_dev: torch.Tensor, inbox: PeerInbox, keep_local: bool):
    """Drive ``batches`` (an iterator of ``(keys, rows)`` on this rank) to the owners under ``owner_dev``:
    rows for other ranks travel as peer copies, rows that stay are inserted locally when ``keep_local``.
    Every rank loops until all ranks are out of batches. Returns (rows received, keys that left)."""
    rank = table.rank
    stride = table.table.stride()
    received, leaving = 0, []
    it = iter(batches)
    while True:
        nxt = next(it, None)
        if not _any_rank(table, nxt is not None):
            break
        if nxt is None:
            keys = torch.empty(0, dtype=torch.int64, device=table.device)
            rows = torch.empty((0, stride), device=table.device)
        else:
            keys, rows = nxt
        dest = route(table, keys, owner_dev).long()
        move = dest != rank
        if keep_local and (~move).any():
            table.set_rows(keys[~move], rows[~move], emb_only=False)
            received += int((~move).sum().item())
        leaving.append(keys[move])
        received += _ship(table, inbox, keys[move], rows[move], dest[move])
    return received, leaving


def _scan_keys(table: SparseTable, mode: int, owner_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Keys of this rank's table that pass an index scan filter, keys only, one kernel: mode 0 = all,
    2 = keys whose shard belongs to another rank under the map ``owner_dev``, 4 = rows changed since the
    dirty bits were last cleared."""
    n_local = table.size()
    buf = torch.empty(max(n_local, 1), dtype=torch.int64, device=table.device)
    st, n, _ = table.table.export_window(0, table.table.index_capacity(), mode, -1, table.rank, table.n_shards,
                                         0 if owner_dev is None else owner_dev.data_ptr(), buf.data_ptr(), 0,
                                         torch.cuda.current_stream().cuda_stream)
    raise_if_error(st)
    return buf[:n]


def exchange_by_keys(source: SparseTable, keys: torch.Tensor, send: List[int], inbox: PeerInbox, target: SparseTable,
                     comm: SparseTable, between_rounds=None) -> int:
    """Ship the rows of ``keys`` (sorted by destination rank, ``send[d]`` of them for rank ``d``) from the
    local table ``source`` into the tables ``target`` of their destinations. Collective over ``comm``'s
    group. The per-pair totals are exchanged once, so every rank knows the whole schedule; per round the
    row-fetch kernel writes up to ``inbox.cap`` rows per destination straight into that rank's inbox
    over NVLink (peer stores) and the destination inserts what arrived. Returns rows received."""
    world, rank = comm.world, comm.rank
    cap = inbox.cap
    stream = torch.cuda.current_stream().cuda_stream
    recv = _exchange_counts(comm, send)
    offs = [0] * world
    for d in range(1, world):
        offs[d] = offs[d - 1] + send[d - 1]
    rounds = (max(send + [0]) + cap - 1) // cap
    if world > 1:
        t = torch.tensor([rounds], device=comm.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=comm.group)
        rounds = int(t.item())
    found = torch.empty(cap, dtype=torch.int32, device=comm.device)
    for i in range(rounds):
        for step in range(world):
            d = (rank + 1 + step) % world          # ring order: the ranks write to different peers at any moment
            n = min(cap, send[d] - i * cap)
            if n > 0:
                ks = keys[offs[d] + i * cap: offs[d] + i * cap + n]
                _, rptr = inbox.region_ptrs(d, rank)
                inbox.keys_view(d, rank)[:n].copy_(ks)
                raise_if_error(source.table.get_rows(ks.data_ptr(), n, rptr, found.data_ptr(), False, stream))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=comm.group)        # every peer store has landed
        for src in range(world):
            n = min(cap, recv[src] - i * cap)
            if n > 0:
                k, r = inbox.received(src, n)
                target.set_rows(k, r, emb_only=False)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=comm.group)        # the inboxes may be overwritten again
        if between_rounds is not None:
            between_rounds()                      # e.g. read-only pulls: the old owners still hold every row
    return sum(recv)


def reshard(table: SparseTable, new_owner: Sequence[int], batch: int = 1 << 18, inbox: Optional[PeerInbox] = None,
            stats: Optional[dict] = None, between_rounds=None) -> int:
    """Move every row whose shard changes hands to its new owner; returns the number of rows this rank
    received. Pulls and pushes must not run concurrently (writes pause, as in the reference). One index
    scan lists the keys that leave, they are sorted by destination and shipped with
    :func:`exchange_by_keys`: the work is proportional to the rows that move, not to the table.
    ``stats`` (optional) receives the host-side duration of each phase in milliseconds. ``between_rounds``
    (optional, collective) runs after every round of the exchange: reads stay served during a migration by
    issuing read-only pulls (``insert=False``) there, since rows are purged from their old owners and the owner
    map is swapped only at the very end, every key is still found where the current map says (the reference keeps
    serving reads during a reshard the same way, pico-ps/handler/UpdateContextHandler.cpp:62-153).

    A table created with ``sync=True``: call ``store()`` before moving rows of a CUDA table. A row travels with its
    pending delta, but the GPU table does not put it on the list that the next ``store`` walks at its new place (the
    host table does)."""
    import time
    if not table.is_cuda:
        return _host.reshard(table, new_owner, stats, between_rounds)
    world = table.world
    marks = []

    def mark(name):
        if stats is not None:
            torch.cuda.synchronize()
            marks.append((name, time.perf_counter()))

    mark("start")
    new_owner = list(new_owner)
    owner_dev = torch.tensor(new_owner, dtype=torch.int32, device=table.device)
    inbox = inbox or PeerInbox(table, batch)
    leaving = _scan_keys(table, 2, owner_dev)
    mark("scan")
    dest = route(table, leaving, owner_dev).long()
    leaving = leaving[torch.argsort(dest, stable=True)]
    send = torch.bincount(dest, minlength=world).tolist()
    mark("sort")
    received = exchange_by_keys(table, leaving, send, inbox, table, table, between_rounds)
    mark("exchange")
    if leaving.numel():
        table.erase_keys(leaving)                  # purge: what moved away no longer belongs here
    mark("purge")
    table.set_shard_owner(new_owner)
    if world > 1:
        dist.barrier(group=table.group)
    mark("swap")
    if stats is not None:
        for (_, t0), (name, t1) in zip(marks, marks[1:]):
            stats[name] = stats.get(name, 0.0) + (t1 - t0) * 1e3
    return received


class ReplicaSet:
    """2x replication for a collective table: rank ``r`` mirrors the shards of rank ``(r - 1) % world`` in a
    second table and ships its own changes to rank ``(r + 1) % world``. For a table on the host back-end the
    constructor hands back the host implementation with the same methods."""

    def __new__(cls, table: SparseTable, batch: int = 1 << 18, in_push: bool = False):
        if not table.is_cuda:
            return _host.HostReplicaSet(table)
        return super().__new__(cls)

    def __init__(self, table: SparseTable, batch: int = 1 << 18, in_push: bool = False):
        """``in_push=True`` (the table must have been created with ``replicate=True``): every fused push also
        applies its row updates to the mirror on the partner GPU from inside the kernel, as the reference's push
        reaches every node that hosts a shard (pico-ps/operator/SparsePushOperator.h:161-168). The mirror is then
        exact after every push and ``sync()`` is only needed for rows that changed by other means (set_rows, load)."""
        self.table = table
        self.in_push = bool(in_push)
        self.world, self.rank = table.world, table.rank
        self.batch = batch
        table.table.enable_dirty_tracking()
        self.mirror = SparseTable(table.dim, table.opt_name, None, capacity=max(1024, table.table.index_capacity() // 2),
                                  max_keys=batch, n_shards=1, sync=table.sync, device=table.device, group="none")
        self.inbox = PeerInbox(table, batch)
        self.partner = (self.rank + 1) % self.world      # holds my mirror
        self.mirrored = (self.rank - 1) % self.world     # whose rows my mirror holds
        self._full_next = True                           # the first sync ships everything
        if self.in_push:
            raise_if_error(table.engine.set_mirror(self.mirror.table))

    def _one_dest(self, n: int, dest: int) -> List[int]:
        send = [0] * self.world
        send[dest] = n
        return send

    def sync(self) -> int:
        """Ship the rows that changed since the last sync (everything, the first time) to the partner's
        mirror. Returns rows sent."""
        t = self.table
        keys = _scan_keys(t, 0 if self._full_next else 4)
        self._full_next = False
        exchange_by_keys(t, keys, self._one_dest(keys.numel(), self.partner), self.inbox, self.mirror, t)
        raise_if_error(t.table.clear_dirty(torch.cuda.current_stream().cuda_stream))
        return int(keys.numel())

    def restore(self, lost_rank: int) -> int:
        """Refill the primary table of ``lost_rank`` (cleared, e.g. after its process was replaced) from
        the mirror kept by its partner. Collective. Returns rows restored on ``lost_rank``."""
        t = self.table
        holder = (lost_rank + 1) % self.world
        if self.rank == holder:
            keys = _scan_keys(self.mirror, 0)
        else:
            keys = torch.empty(0, dtype=torch.int64, device=t.device)
        return exchange_by_keys(self.mirror, keys, self._one_dest(keys.numel(), lost_rank), self.inbox, t, t)
