"""Host back-end of shard migration, replica sync and restore: the same collective calls as ``migrate.py`` for
tables that live in :class:`HostTable` storage (``device="cpu"``), with the rows carried by object collectives of
the process group (gloo) instead of NVLink peer copies. It exists so that the elastic logic (which rows leave, when
the owner map is swapped, what a mirror holds) runs and is tested on machines without a GPU; it is not a fast path.

The transaction is the one of the GPU path and of the reference (pico-ps/handler/UpdateContextHandler.cpp:62-153):
new shards are created on their new owners, rows are shuffled, the old owners drop the shards that left, the owner
map is swapped last.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from .._lib import C
from ..ops.sparse import SparseTable

Part = Tuple[np.ndarray, np.ndarray]


def shards_of(table: SparseTable, keys: torch.Tensor, owner: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Shard of every key, or the owning rank under the map ``owner``."""
    out = C.sparse_shards_of(keys.reshape(-1).cpu().numpy(), table.n_shards, list(owner) if owner is not None else [])
    return torch.from_numpy(out)


def _empty(stride: int) -> Part:
    return np.empty(0, dtype=np.int64), np.empty((0, stride), dtype=np.float32)


def all_to_all_rows(table: SparseTable, parts: List[Part]) -> List[Part]:
    """``parts[d]`` goes to rank ``d``; returns what every rank sent to this one, by source rank."""
    if table.world == 1:
        return [parts[0]]
    gathered = [None] * table.world
    dist.all_gather_object(gathered, parts, group=table.group)
    return [gathered[src][table.rank] for src in range(table.world)]


def split_by_dest(keys: torch.Tensor, rows: torch.Tensor, dest: torch.Tensor, world: int, stride: int) -> List[Part]:
    k, r, d = keys.cpu().numpy(), rows.cpu().numpy().reshape(-1, stride), dest.cpu().numpy()
    return [(k[d == w], r[d == w]) if len(k) else _empty(stride) for w in range(world)]


def ship(table: SparseTable, keys: torch.Tensor, rows: torch.Tensor, dest: torch.Tensor,
         target: Optional[SparseTable] = None) -> int:
    """Send (keys, rows) to the ranks in ``dest`` and insert what this rank receives into ``target``."""
    target = target or table
    stride = table.table.stride()
    got = all_to_all_rows(table, split_by_dest(keys, rows, dest, table.world, stride))
    total = 0
    for k, r in got:
        if len(k):
            target.set_rows(torch.from_numpy(k), torch.from_numpy(r), emb_only=False)
            total += len(k)
    return total


def _export_all(table: SparseTable, shards: Sequence[int], dirty_only: bool = False) -> Part:
    ks, rs = [], []
    for s in shards:
        for k, r in table.export(shard=s, dirty_only=dirty_only):
            ks.append(k.numpy())
            rs.append(r.numpy())
    if not ks:
        return _empty(table.table.stride())
    return np.concatenate(ks), np.concatenate(rs)


def reshard(table: SparseTable, new_owner: Sequence[int], stats: Optional[dict] = None, between_rounds=None) -> int:
    """Collective. Moves every shard whose owner changes; returns the rows this rank received."""
    new_owner = list(new_owner)
    old_owner = list(table.shard_owner)
    if len(new_owner) != table.n_shards or any(not 0 <= o < table.world for o in new_owner):
        raise ValueError("new_owner needs one rank in [0, world) per shard")
    rank, world, stride = table.rank, table.world, table.table.stride()
    arriving = [s for s in range(table.n_shards) if new_owner[s] == rank and old_owner[s] != rank]
    leaving = [s for s in range(table.n_shards) if old_owner[s] == rank and new_owner[s] != rank]
    for s in arriving:
        if not table.table.has_shard(s):
            table.table.create_shard(s)
    parts = [_empty(stride) for _ in range(world)]
    by_dest = {}
    for s in leaving:
        by_dest.setdefault(new_owner[s], []).append(s)
    for d, shards in by_dest.items():
        parts[d] = _export_all(table, shards)
    received = 0
    for k, r in all_to_all_rows(table, parts):
        if len(k):
            table.set_rows(torch.from_numpy(k), torch.from_numpy(r), emb_only=False)
            received += len(k)
    if between_rounds is not None:
        between_rounds()                     # the old owners still hold every row and the old map still routes
    for s in leaving:
        table.table.erase_shard(s)           # purge
    table.set_shard_owner(new_owner)
    if world > 1:
        dist.barrier(group=table.group)
    if stats is not None:
        stats["moved_shards"] = stats.get("moved_shards", 0) + len(leaving)
    return received


class HostReplicaSet:
    """2x replication of a host table: rank ``r`` mirrors the rows of rank ``(r - 1) % world`` in a second table
    and ships its own changes (dirty rows; everything the first time) to rank ``(r + 1) % world``."""

    def __init__(self, table: SparseTable):
        self.table = table
        self.world, self.rank = table.world, table.rank
        table.table.enable_dirty_tracking()
        self.mirror = SparseTable(table.dim, table.opt_name, None, n_shards=1, sync=table.sync, device="cpu", group="none")
        self.partner = (self.rank + 1) % self.world
        self.mirrored = (self.rank - 1) % self.world
        self._full_next = True

    def _send_to(self, dest: int, part: Part, target: SparseTable) -> int:
        stride = self.table.table.stride()
        parts = [_empty(stride) for _ in range(self.world)]
        parts[dest] = part
        n = 0
        for k, r in all_to_all_rows(self.table, parts):
            if len(k):
                target.set_rows(torch.from_numpy(k), torch.from_numpy(r), emb_only=False)
                n += len(k)
        return n

    def sync(self) -> int:
        t = self.table
        part = _export_all(t, t.table.shard_list(), dirty_only=not self._full_next)
        self._full_next = False
        self._send_to(self.partner, part, self.mirror)
        t.table.clear_dirty()
        return len(part[0])

    def restore(self, lost_rank: int) -> int:
        """Refill the (cleared) primary table of ``lost_rank`` from the mirror its partner keeps. Collective."""
        holder = (lost_rank + 1) % self.world
        part = _export_all(self.mirror, self.mirror.table.shard_list()) if self.rank == holder \
            else _empty(self.table.table.stride())
        return self._send_to(lost_rank, part, self.table)
