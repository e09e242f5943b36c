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
from ..ops.dedup import KeyDeduper
from ..ops.dense import _view
from ..ops.sparse import SparseTable
from ..utils.status import raise_if_error


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


def reshard(table: SparseTable, new_owner: Sequence[int], batch: int = 1 << 18) -> int:
    """Move every row whose shard changes hands to its new owner; returns the number of rows this rank
    received. Pulls and pushes must not run concurrently (writes pause, as in the reference)."""
    world, rank = table.world, table.rank
    new_owner = list(new_owner)
    owner_dev = torch.tensor(new_owner, dtype=torch.int32, device=table.device)
    inbox = PeerInbox(table, batch)
    dedup = KeyDeduper(batch, table.device)
    received = 0
    # export in windows so that one batch fits the inbox; every rank loops the same number of times
    batches = list(table.export(batch=batch))
    n_rounds = len(batches)
    if world > 1:
        t = torch.tensor([n_rounds], device=table.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=table.group)
        n_rounds = int(t.item())
    leaving: List[torch.Tensor] = []
    for i in range(n_rounds):
        if i < len(batches):
            keys, rows = batches[i]
            _, owner, inverse, _ = dedup(keys, owner_dev, world)
            dest = owner[inverse.long()].long()
            move = dest != rank
            leaving.append(keys[move])
            received += _ship(table, inbox, keys[move], rows[move], dest[move])
        else:
            empty_k = torch.empty(0, dtype=torch.int64, device=table.device)
            empty_r = torch.empty((0, table.table.stride()), device=table.device)
            received += _ship(table, inbox, empty_k, empty_r, torch.empty(0, dtype=torch.int64, device=table.device))
    for k in leaving:
        if k.numel():
            table.erase_keys(k)       # purge: what moved away no longer belongs here
    table.set_shard_owner(new_owner)
    if world > 1:
        dist.barrier(group=table.group)
    return received


class ReplicaSet:
    """2x replication for a collective table: rank ``r`` mirrors the shards of rank ``(r - 1) % world`` in a
    second table and ships its own changes to rank ``(r + 1) % world``."""

    def __init__(self, table: SparseTable, batch: int = 1 << 18):
        self.table = table
        self.world, self.rank = table.world, table.rank
        self.batch = batch
        table.table.enable_dirty_tracking()
        self.mirror = SparseTable(table.dim, table.opt_name, None, capacity=max(1024, table.table.index_capacity() // 2),
                                  max_keys=batch, n_shards=1, sync=table.sync, device=table.device, group="none")
        self.inbox = PeerInbox(table, batch)
        self.partner = (self.rank + 1) % self.world      # holds my mirror
        self.mirrored = (self.rank - 1) % self.world     # whose rows my mirror holds
        self._full_next = True                           # the first sync ships everything

    def _rounds(self, n_local: int) -> int:
        if self.world == 1:
            return n_local
        t = torch.tensor([n_local], device=self.table.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.table.group)
        return int(t.item())

    def sync(self) -> int:
        """Ship the rows that changed since the last sync (everything, the first time) to the partner's
        mirror. Returns rows sent."""
        t = self.table
        batches = list(t.export(batch=self.batch, dirty_only=not self._full_next))
        self._full_next = False
        sent = 0
        for i in range(self._rounds(len(batches))):
            if i < len(batches):
                keys, rows = batches[i]
            else:
                keys = torch.empty(0, dtype=torch.int64, device=t.device)
                rows = torch.empty((0, t.table.stride()), device=t.device)
            dest = torch.full((keys.numel(),), self.partner, dtype=torch.int64, device=t.device)
            _ship(t, self.inbox, keys, rows, dest, target=self.mirror)
            sent += keys.numel()
        raise_if_error(t.table.clear_dirty(torch.cuda.current_stream().cuda_stream))
        return sent

    def restore(self, lost_rank: int) -> int:
        """Refill the primary table of ``lost_rank`` (cleared, e.g. after its process was replaced) from
        the mirror kept by its partner. Collective. Returns rows restored on ``lost_rank``."""
        t = self.table
        holder = (lost_rank + 1) % self.world
        batches = list(self.mirror.export(batch=self.batch)) if self.rank == holder else []
        got = 0
        for i in range(self._rounds(len(batches))):
            if i < len(batches):
                keys, rows = batches[i]
            else:
                keys = torch.empty(0, dtype=torch.int64, device=t.device)
                rows = torch.empty((0, t.table.stride()), device=t.device)
            dest = torch.full((keys.numel(),), lost_rank, dtype=torch.int64, device=t.device)
            got += _ship(t, self.inbox, keys, rows, dest)
        return got
