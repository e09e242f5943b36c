"""Stand-alone key dedup + partition (``csrc/kernels/dedup.cu``): distinct keys, inverse map, owner of
every distinct key and per-owner counts. The client-side step of a sparse request
(pico-ps/operator/SparsePullOperator.h:91-101) for callers that route requests themselves."""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from .._lib import C


class KeyDeduper:
    """Owns the scratch table for batches of up to ``max_keys`` keys."""

    def __init__(self, max_keys: int, device=None):
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.max_keys = int(max_keys)
        slots = 1
        while slots < 2 * self.max_keys:
            slots <<= 1
        self.slots = slots
        self.scratch = torch.empty(slots * 16, dtype=torch.uint8, device=self.device)
        self.pos = torch.empty(self.max_keys, dtype=torch.int32, device=self.device)
        self._refill()

    def _refill(self) -> None:
        rc = C.dedup_fill_scratch(self.scratch.data_ptr(), self.slots, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"dedup_fill_scratch failed: {rc}")

    def __call__(self, keys: torch.Tensor, shard_owner: Optional[torch.Tensor] = None, world: int = 1
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """Returns ``(unique_keys, unique_owner, inverse, counts)``; ``counts[0]`` is the number of distinct
        keys, ``counts[1 + r]`` how many of them rank ``r`` owns. ``shard_owner`` is an int32 tensor
        ``[n_shards]`` (absent: everything belongs to rank 0)."""
        if keys.dtype != torch.int64 or not keys.is_cuda:
            raise TypeError("keys must be a CUDA int64 tensor")           # a host pointer must never reach the kernel
        if shard_owner is not None and (shard_owner.dtype != torch.int32 or not shard_owner.is_cuda or not shard_owner.is_contiguous()):
            raise TypeError("shard_owner must be a contiguous CUDA int32 tensor")
        if world < 1:
            raise ValueError("world must be at least 1")
        keys = keys.reshape(-1).contiguous()
        n = keys.numel()
        if n > self.max_keys:
            raise ValueError("batch larger than max_keys")
        uniq = torch.empty(n, dtype=torch.int64, device=self.device)
        owner = torch.empty(n, dtype=torch.int32, device=self.device)
        inverse = torch.empty(n, dtype=torch.int32, device=self.device)
        counts = torch.empty(1 + world, dtype=torch.int32, device=self.device)
        n_shards = 0 if shard_owner is None else shard_owner.numel()
        rc = C.dedup_partition(keys.data_ptr(), n, self.scratch.data_ptr(), self.slots, self.pos.data_ptr(),
                               0 if shard_owner is None else shard_owner.data_ptr(), n_shards, world, uniq.data_ptr(),
                               owner.data_ptr(), inverse.data_ptr(), counts.data_ptr(),
                               torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"dedup_partition failed: {rc}")
        nu = int(counts[0].item())
        if nu < 0:   # bit 31: the error mark of the kernels
            self._refill()
            raise ValueError("dedup_partition: a key equals a reserved value (INT64_MIN, INT64_MIN + 1), a shard owner is "
                             "outside [0, world), or the scratch table was in use by an overlapping call")
        return uniq[:nu], owner[:nu], inverse, counts
