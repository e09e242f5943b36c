"""The switches of the GPU kernels exist on the host back-end too (as no-ops), so that a script written for a GPU
job runs unchanged on CPU, and the host restatement of the reproducible push's summation order is what it says."""
import numpy as np
import pytest
import torch

from blocked_sum import BLOCK, blocked_segment_sum
from parameter_server_b200 import SparseTable
from parameter_server_b200.ops.dense import DenseTable


def test_gpu_only_switches_are_accepted_by_host_tables():
    t = SparseTable(8, "adagrad", dict(lr=0.1), device="cpu", group="none")
    t.set_sm_budget(4, 4)
    t.set_grad_wire_bf16(True)
    t.set_deterministic(True)
    k = torch.arange(10)
    assert t.pull(k).shape == (10, 8)
    t.push(torch.ones(10, 8))
    assert t.size() == 10
    d = DenseTable({"w": (4, 4)}, "sgd", dict(lr=0.1), device="cpu", group="none")
    d.set_sm_budget(3)


def test_blocked_sum_is_a_plain_left_to_right_sum_up_to_one_block():
    rng = np.random.default_rng(0)
    keys = rng.integers(0, 50, size=2000)
    grads = (rng.standard_normal((2000, 4)) * 1e3).astype(np.float32)
    uniq, agg = blocked_segment_sum(keys, grads)
    for i, u in enumerate(uniq):
        rows = grads[keys == u]
        if len(rows) <= BLOCK:
            acc = np.zeros(4, dtype=np.float32)
            for r in rows:
                acc = acc + r
            assert np.array_equal(acc, agg[i])
    # a key with more than one block: block sums first, then the blocks in order
    keys = np.zeros(3 * BLOCK + 5, dtype=np.int64)
    grads = (rng.standard_normal((len(keys), 2)) * 1e3).astype(np.float32)
    _, agg = blocked_segment_sum(keys, grads)
    parts = []
    for b in range(0, len(keys), BLOCK):
        acc = np.zeros(2, dtype=np.float32)
        for r in grads[b:b + BLOCK]:
            acc = acc + r
        parts.append(acc)
    tot = np.zeros(2, dtype=np.float32)
    for p_ in parts:
        tot = tot + p_
    assert np.array_equal(tot, agg[0])


def test_misuse_is_answered_with_an_exception_not_with_silent_damage():
    import numpy as np
    from parameter_server_b200 import SparseTable
    from parameter_server_b200.ops.dense import DenseTable
    d = DenseTable({"w": (4, 4), "b": (4,)}, "adamw", dict(lr=1e-2), device="cpu")
    with pytest.raises(ValueError):
        d.load({"w": torch.ones(5, 5)})                      # would have run over the neighbour's parameters
    with pytest.raises(KeyError):
        d.load({"zzz": torch.ones(4)})
    d.load({"w": torch.ones(4, 4)})
    assert float(d.pull("w").sum()) == 16.0 and float(d.pull("b").abs().sum()) == 0.0
    with pytest.raises(ValueError):
        SparseTable(8, "sgd", dict(lr=0.1), device="cpu", group="none", n_shards=-1)
    t = SparseTable(8, "sgd", dict(lr=0.1), device="cpu", group="none")
    t.pull(torch.arange(50))
    # a scan cursor always moves on, whatever window the caller asks for
    k, r, cursor, finished = t.table.export_shard(0, 0, 0, False)
    assert cursor == 1 and not finished
    k, r, cursor, finished = t.table.export_shard(0, 1 << 60, 10, False)
    assert finished and len(k) == 0
