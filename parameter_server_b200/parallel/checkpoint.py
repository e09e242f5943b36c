"""Dump / load of a collective-path :class:`SparseTable` in the layout of the RPC path's DumpOperator.

``dump(table, uri, file_number)`` writes ``<uri>/model_<rank>_<file>``; a record goes to file
``shard % file_number`` of the rank that holds it (pico-ps/operator/DumpOperator.h:109-147). Files are
in the binary record codec of ``csrc/operator/operators.h`` (header ``PSB1`` + u32 record width, then
``int64 key, width * fp32`` per record), so dumps written by the RPC servers and by the collective path
load into each other. ``load(table, uri)`` re-hashes: the ranks split the files of the directory
between them, whatever number of nodes wrote them, and route every record to its owner under the
table's current shard map as NVLink peer copies (pico-ps/operator/LoadOperator.h:87-143).

``uri`` may also name a directory of a Hadoop file system (``hdfs://...``): the files are then staged through a local
temporary directory and moved with the ``hadoop`` command configured for the service layer
(``service.set_hadoop_bin`` / ``$PSB_HADOOP_BIN``), the same way the RPC servers reach such paths.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import tempfile
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..ops.sparse import SparseTable
from .migrate import PeerInbox, route, stream_to_owners

_MAGIC = b"PSB1"
_REMOTE = ("hdfs://", "viewfs://", "s3a://", "gs://", "abfs://")


def _is_remote(path: str) -> bool:
    return path.startswith(_REMOTE)


def _hadoop(*args: str, capture: bool = False) -> str:
    from .._lib import C
    p = subprocess.run([C.hadoop_bin(), "fs", *args], capture_output=capture, text=capture)
    if p.returncode != 0:
        raise RuntimeError(f"hadoop fs {' '.join(args)} failed with exit code {p.returncode}")
    return p.stdout if capture else ""


def _record_dtype(stride: int) -> np.dtype:
    return np.dtype([("key", "<i8"), ("row", "<f4", (stride,))])


def dump(table: SparseTable, uri: str, file_number: int = 1, batch: int = 1 << 18) -> int:
    """Collective. Returns the number of records this rank wrote."""
    target = uri.split("?", 1)[0]
    if not target:
        raise ValueError("dump: the uri names no directory")
    if int(file_number) < 1:
        raise ValueError("dump: file_number must be at least 1")
    remote = _is_remote(target)
    path = tempfile.mkdtemp(prefix="psb_dump_") if remote else target
    os.makedirs(path, exist_ok=True)
    stride = table.table.stride()
    rec = _record_dtype(stride)
    files = []
    for f in range(file_number):
        fh = open(os.path.join(path, f"model_{table.rank}_{f}"), "wb")
        fh.write(_MAGIC + np.uint32(stride).tobytes())
        files.append(fh)
    written = 0
    for keys, rows in table.export(batch=batch):
        which = (route(table, keys, None) % file_number).cpu().numpy()
        k, r = keys.cpu().numpy(), rows.cpu().numpy()
        for f in range(file_number):
            sel = which == f
            m = int(sel.sum())
            if m:
                block = np.empty(m, dtype=rec)
                block["key"], block["row"] = k[sel], r[sel]
                block.tofile(files[f])
                written += m
    for fh in files:
        fh.close()
    if remote:
        try:
            _hadoop("-mkdir", "-p", target)
            for f in range(file_number):
                name = f"model_{table.rank}_{f}"
                _hadoop("-put", "-f", os.path.join(path, name), f"{target}/{name}")
        finally:
            shutil.rmtree(path, ignore_errors=True)
    if table.world > 1:
        dist.barrier(group=table.group)
    return written


def _read_batches(paths, stride: int, batch: int, device):
    rec = _record_dtype(stride)
    for p in paths:
        with open(p, "rb") as fh:
            head = fh.read(8)
            if head[:4] != _MAGIC or int(np.frombuffer(head[4:], dtype="<u4")[0]) != stride:
                raise RuntimeError(f"{p}: not a PSB1 dump of record width {stride}")
            while True:
                block = np.fromfile(fh, dtype=rec, count=batch)
                if block.size == 0:
                    break
                yield (torch.from_numpy(np.ascontiguousarray(block["key"])).to(device),
                       torch.from_numpy(np.ascontiguousarray(block["row"])).to(device))


def _damaged(paths, stride: int) -> Optional[str]:
    """The first file that is not an intact dump of this record width (header, whole records), or None."""
    rec_bytes = _record_dtype(stride).itemsize
    for p in paths:
        size = os.path.getsize(p)
        with open(p, "rb") as fh:
            head = fh.read(8)
        if len(head) < 8 or head[:4] != _MAGIC or int(np.frombuffer(head[4:8], dtype="<u4")[0]) != stride:
            return f"{p}: not a PSB1 dump of record width {stride}"
        if (size - 8) % rec_bytes:
            return f"{p}: truncated (the last record is cut short)"
    return None


def load(table: SparseTable, uri: str, batch: int = 1 << 18, inbox: Optional[PeerInbox] = None,
         only_node: Optional[int] = None) -> int:
    """Collective. Inserts every record of the dump at ``uri`` (of the files written by ``only_node`` when
    given: the restore of one lost rank) into its owner's table; existing rows are overwritten. Returns
    the number of records that landed on this rank."""
    path = uri.split("?", 1)[0]
    prefix = "model_" if only_node is None else f"model_{only_node}_"
    staged = None
    if _is_remote(path):
        listing = _hadoop("-ls", path, capture=True).splitlines()
        names = sorted(line.rsplit("/", 1)[1] for line in listing if line[:1] in "-d" and "/" in line)
        names = [n for n in names if n.startswith(prefix)]
        staged = tempfile.mkdtemp(prefix="psb_load_")
        mine = []
        for n in names[table.rank::table.world]:          # every rank fetches only the files it will read
            _hadoop("-get", f"{path}/{n}", os.path.join(staged, n))
            mine.append(os.path.join(staged, n))
    else:
        names = sorted(n for n in os.listdir(path) if n.startswith(prefix))
        mine = [os.path.join(path, n) for n in names[table.rank::table.world]]
    # every rank checks its files BEFORE the collective part and the ranks agree on the verdict: a rank that
    # raised alone would leave the others waiting in a collective
    problem = _damaged(mine, table.table.stride())
    flag = torch.tensor([1 if problem else 0], device=table.device)
    if table.world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=table.group)
    if int(flag.item()):
        raise RuntimeError(problem or "load: another rank found a damaged dump file")
    owner_dev = torch.tensor(table.shard_owner, dtype=torch.int32, device=table.device)
    if table.is_cuda:
        inbox = inbox or PeerInbox(table, batch)
    got, _ = stream_to_owners(table, _read_batches(mine, table.table.stride(), batch, table.device), owner_dev, inbox,
                              keep_local=True)
    if staged is not None:
        shutil.rmtree(staged, ignore_errors=True)
    if table.world > 1:
        dist.barrier(group=table.group)
    return got
