"""Host restatement of the summation order of the reproducible push (csrc/kernels/segment_sum.h): the occurrences of
a key, in position order, are cut into blocks of 64; every block is added front to back, then the block sums are
added front to back. fp32 throughout, one add at a time (``np.add.at`` is sequential in the order it is given)."""
import numpy as np

BLOCK = 64


def blocked_segment_sum(keys: np.ndarray, grads: np.ndarray):
    """Returns (unique keys ascending, their summed gradient rows)."""
    keys = np.asarray(keys)
    grads = np.asarray(grads, dtype=np.float32)
    uniq, inv = np.unique(keys, return_inverse=True)
    order = np.argsort(inv, kind="stable")                 # by key, position order inside a key
    s_inv = inv[order]
    n = len(keys)
    starts = np.r_[0, np.flatnonzero(np.diff(s_inv)) + 1]
    lens = np.diff(np.r_[starts, n])
    rank = np.arange(n) - np.repeat(starts, lens)          # occurrence number inside the key
    blk = rank // BLOCK
    nblk = int(blk.max()) + 1 if n else 1
    kb = s_inv.astype(np.int64) * nblk + blk               # (key, block), already ascending
    ukb, kb_inv = np.unique(kb, return_inverse=True)
    part = np.zeros((len(ukb), grads.shape[1]), dtype=np.float32)
    np.add.at(part, kb_inv, grads[order])                  # level 1: inside a block, front to back
    agg = np.zeros((len(uniq), grads.shape[1]), dtype=np.float32)
    np.add.at(agg, (ukb // nblk).astype(np.int64), part)   # level 2: the blocks of a key, front to back
    return uniq, agg
