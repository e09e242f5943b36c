"""Synthetic key batches for the benchmarks."""
from __future__ import annotations

import numpy as np


def zipf_batch(rng: np.random.Generator, n: int, s: float, vocab: int, min_duplicate_rate: float = 0.0) -> np.ndarray:
    """``n`` int64 keys in ``[0, vocab)``: Zipf(``s``) ranks scattered over the key space by a multiplicative
    hash. If fewer than ``min_duplicate_rate`` of the positions repeat another key of the batch, more
    positions are overwritten with copies of random other positions until that rate is reached."""
    z = rng.zipf(s, size=n).astype(np.uint64)
    k = (((z * np.uint64(0x9E3779B97F4A7C15)) >> np.uint64(1)) % np.uint64(vocab)).astype(np.int64)
    if min_duplicate_rate > 0:
        dup = 1.0 - np.unique(k).size / n
        if dup < min_duplicate_rate:
            sel = rng.random(n) < (min_duplicate_rate - dup) / max(1e-9, 1.0 - dup)
            k[sel] = k[rng.integers(0, n, size=int(sel.sum()))]
    return k
