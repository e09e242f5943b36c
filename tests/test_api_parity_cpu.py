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


@pytest.mark.parametrize("opt,kw", [("adamw", dict(lr=1e-2, weight_decay=0.01)), ("sgd", dict(lr=0.1)), ("adagrad", dict(lr=0.1))])
def test_a_dense_table_resumes_from_its_checkpoint_exactly(tmp_path, opt, kw):
    """`checkpoint.dump_dense / load_dense`: master values, optimizer slots and the step count come back, so the next
    step of the resumed table is the next step of the original; a checkpoint of other tensors or of another optimizer
    is refused."""
    from parameter_server_b200.parallel import checkpoint
    shapes = {"w": (33, 7), "b": (33,), "g": (5,)}
    a = DenseTable(shapes, opt, kw, device="cpu", group="none")
    gen = torch.Generator().manual_seed(3)
    a.load({"w": torch.randn(33, 7, generator=gen), "b": torch.randn(33, generator=gen), "g": torch.ones(5)})
    for _ in range(3):
        a.zero_grads()
        a.grads["w"].add_(torch.randn(33, 7, generator=gen))
        a.grads["b"].add_(0.1)
        a.push()
    n = checkpoint.dump_dense(a, str(tmp_path))
    assert n == a.numel and sorted(p.name for p in tmp_path.iterdir()) == ["dense_0.npz"]
    b = DenseTable(shapes, opt, kw, device="cpu", group="none")
    assert checkpoint.load_dense(b, str(tmp_path)) == n and b.step_count == a.step_count == 3
    g = torch.randn(33, 7, generator=gen)
    for t in (a, b):
        t.zero_grads()
        t.grads["w"].add_(g)
        t.push()
    assert all(torch.equal(a.pull(k), b.pull(k)) for k in shapes)
    with pytest.raises(RuntimeError):
        checkpoint.load_dense(DenseTable({"w": (33, 7)}, opt, kw, device="cpu", group="none"), str(tmp_path))
    other = "sgd" if opt != "sgd" else "adagrad"
    with pytest.raises(RuntimeError):
        checkpoint.load_dense(DenseTable(shapes, other, dict(lr=0.1), device="cpu", group="none"), str(tmp_path))
    with pytest.raises(FileNotFoundError):
        checkpoint.load_dense(b, str(tmp_path / "nothing_here"))
