"""The allocation-free dedup entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory at the point where they need the
operation (a serving loop with a fixed memory budget, a plug-in that only gets buffers from its
host application), so ``psb_dedup_partition_noalloc`` keeps its scratch in a fixed array inside the
library. The test calls it twice in a row through ``ctypes`` and checks every output against the
regular entry point (``KeyDeduper``), which allocates its scratch with torch. Collected last on
purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from parameter_server_b200 import C, _build
from parameter_server_b200.ops.dedup import KeyDeduper

pytestmark = pytest.mark.gpu

MAX_KEYS = 65536


def _entry():
    lib = ctypes.CDLL(str(_build.lib_path()))
    fn = lib.psb_dedup_partition_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _call(fn, keys, shard_owner, world):
    n = keys.numel()
    uniq = torch.empty(max(n, 1), dtype=torch.int64, device="cuda")
    owner = torch.empty(max(n, 1), dtype=torch.int32, device="cuda")
    inverse = torch.empty(max(n, 1), dtype=torch.int32, device="cuda")
    counts = torch.empty(1 + world, dtype=torch.int32, device="cuda")
    rc = fn(keys.data_ptr(), n, shard_owner.data_ptr(), shard_owner.numel(), world, uniq.data_ptr(), owner.data_ptr(),
            inverse.data_ptr(), counts.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, uniq, owner, inverse, counts


def test_noalloc_matches_regular_entry_point_twice():
    fn = _entry()
    world, n_shards = 4, 11
    shard_owner = torch.tensor([s % world for s in range(n_shards)], dtype=torch.int32, device="cuda")
    regular = KeyDeduper(MAX_KEYS)
    rng = np.random.default_rng(5)
    for round_ in range(2):   # the second call reuses the library's scratch array after the first
        n = (40000, MAX_KEYS)[round_]
        keys = torch.from_numpy((rng.zipf(1.1, size=n).astype(np.int64) * 104729) % 1000003).cuda()
        rc, uniq, owner, inverse, counts = _call(fn, keys, shard_owner, world)
        assert rc == 0
        r_uniq, r_owner, r_inverse, r_counts = regular(keys, shard_owner, world)
        nu = int(counts[0])
        assert nu == r_uniq.numel() and torch.equal(counts, r_counts)
        # the order of distinct keys is an artefact of scheduling: compare as sets and through the inverse map
        assert torch.equal(torch.sort(uniq[:nu])[0], torch.sort(r_uniq)[0])
        assert torch.equal(uniq[:nu][inverse.long()], keys)
        assert torch.equal(uniq[:nu][inverse.long()], r_uniq[r_inverse.long()])
        order, r_order = torch.argsort(uniq[:nu]), torch.argsort(r_uniq)
        assert torch.equal(owner[:nu][order], r_owner[r_order])


def test_noalloc_rejects_oversized_and_bad_arguments():
    fn = _entry()
    shard_owner = torch.zeros(1, dtype=torch.int32, device="cuda")
    keys = torch.zeros(MAX_KEYS + 1, dtype=torch.int64, device="cuda")
    rc, *_ = _call(fn, keys, shard_owner, 1)
    assert rc == -10                       # PSB_DEDUP_ERR_TOO_LARGE
    rc, *_ = _call(fn, keys[:10], shard_owner, 99)
    assert rc == -11                       # PSB_DEDUP_ERR_BAD_ARGUMENT
