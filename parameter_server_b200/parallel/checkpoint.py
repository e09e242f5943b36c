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


# ---- dense tables -----------------------------------------------------------------------------------
# A dense table is cut into one contiguous slice per rank; the owner of a slice holds its fp32 master values and its
# optimizer slots. A checkpoint is that, rank by rank: <uri>/dense_<rank>.npz = {lo, numel, world, step_count,
# optimizer, master[len], slot0[len], slot1[len], layout (names, offsets, shapes as JSON)}. A load puts the slices
# back together and cuts them again for the world that reads them, so a job may resume on another number of GPUs.
# The reference dumps dense tables through the same operators as sparse ones (slices are records of a table with the
# dense partitioner, pico-ps/operator/DumpOperator.h:116-202); the RPC path here does the same. This is the
# collective path's form, where the slices never were records.
def _dense_local_state(table):
    import json
    from .._lib import C
    n_slots = int(C.opt_num_slots(table.opt.type))
    if table.is_cuda:
        lo, length = int(table.engine.shard_lo()), int(table.engine.shard_len())
        torch.cuda.current_stream().synchronize()
        master = table.master.detach().cpu().numpy().copy()
        slots = []
        for s in range(n_slots):
            from ..ops.dense import _view
            slots.append(_view(table.engine.slot_ptr(s), length, torch.float32, table.device, table.engine).cpu().numpy().copy())
    else:
        length = table.numel // table.world
        lo = length * table.rank
        if table.rank == table.world - 1:
            length = table.numel - lo
        master = table.flat_master[lo:lo + length].numpy().copy()
        slots = [t[lo:lo + length].numpy().copy() for t in (table._m, table._v)[:n_slots]]
    layout = json.dumps({n: [int(off), [int(d) for d in shape]] for n, (off, shape) in table.offsets.items()})
    return lo, length, master, slots, layout


def dump_dense(table, uri: str) -> int:
    """Collective. Every rank writes the slice it owns (fp32 master values, optimizer slots, step count) to
    ``<uri>/dense_<rank>.npz``. Returns the number of elements this rank wrote."""
    path = uri.split("?", 1)[0]
    if not path:
        raise ValueError("dump_dense: the uri names no directory")
    if _is_remote(path):
        raise ValueError("dump_dense writes to a local directory")
    os.makedirs(path, exist_ok=True)
    lo, length, master, slots, layout = _dense_local_state(table)
    tmp = os.path.join(path, f".dense_{table.rank}.tmp.npz")
    np.savez(tmp, lo=np.int64(lo), numel=np.int64(table.numel), world=np.int64(table.world),
             step_count=np.int64(table.step_count), opt_type=np.int64(table.opt.type), layout=np.array(layout),
             master=master, **{f"slot{i}": s for i, s in enumerate(slots)})
    os.replace(tmp, os.path.join(path, f"dense_{table.rank}.npz"))      # never a torn file under the final name
    if table.world > 1:
        dist.barrier(group=table.group)
    return int(length)


def load_dense(table, uri: str) -> int:
    """Collective. Reads the slices that ``dump_dense`` wrote - by any number of ranks - and installs values,
    optimizer slots and the step count in ``table``; the tensor names and shapes must be the table's. Returns the
    number of elements of the checkpoint."""
    import json
    from .._lib import C
    path = uri.split("?", 1)[0]
    names = sorted(n for n in os.listdir(path) if n.startswith("dense_") and n.endswith(".npz"))
    if not names:
        raise FileNotFoundError(f"no dense_<rank>.npz under {path}")
    parts = [np.load(os.path.join(path, n), allow_pickle=False) for n in names]
    world0 = int(parts[0]["world"])
    if len(parts) != world0 or sorted(int(p["lo"]) for p in parts) != sorted({int(p["lo"]) for p in parts}):
        raise RuntimeError(f"{path}: the checkpoint was written by {world0} ranks, {len(parts)} slices are here")
    mine = {n: [int(off), [int(d) for d in shape]] for n, (off, shape) in table.offsets.items()}
    if json.loads(str(parts[0]["layout"])) != mine:
        raise RuntimeError(f"{path}: the checkpoint holds other tensors than this table")
    if int(parts[0]["opt_type"]) != int(table.opt.type):
        raise RuntimeError(f"{path}: the checkpoint was written with another optimizer")
    n_slots = int(C.opt_num_slots(table.opt.type))
    total = max(int(p["lo"]) + len(p["master"]) for p in parts)
    full = [np.zeros(max(total, table.numel), dtype=np.float32) for _ in range(1 + n_slots)]
    covered = 0
    for p in parts:
        lo, m = int(p["lo"]), p["master"]
        full[0][lo:lo + len(m)] = m
        for i in range(n_slots):
            full[1 + i][lo:lo + len(m)] = p[f"slot{i}"]
        covered += len(m)
    if covered != total:
        raise RuntimeError(f"{path}: the slices do not cover the table ({covered} of {total} elements)")
    table.step_count = int(parts[0]["step_count"])
    if table.is_cuda:
        from ..ops.dense import _view
        from ..utils.status import raise_if_error
        dev = torch.from_numpy(full[0][:table.numel]).to(table.device)
        stream = torch.cuda.current_stream()
        raise_if_error(table.engine.load_full(dev.data_ptr(), stream.cuda_stream))
        lo, length = int(table.engine.shard_lo()), int(table.engine.shard_len())
        for i in range(n_slots):
            _view(table.engine.slot_ptr(i), length, torch.float32, table.device, table.engine).copy_(
                torch.from_numpy(full[1 + i][lo:lo + length]).to(table.device))
        stream.synchronize()
    else:
        table.flat_master.copy_(torch.from_numpy(full[0][:table.numel]))
        for i, t in enumerate((table._m, table._v)[:n_slots]):
            t.copy_(torch.from_numpy(full[1 + i][:table.numel]))
    if table.world > 1:
        dist.barrier(group=table.group)
    return int(total)
