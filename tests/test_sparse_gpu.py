"""Single-GPU fused pull / push against the CPU oracle (plain fp32 reference of the same op)."""
import os
import numpy as np
import pytest
import torch

from parameter_server_b200 import C, SparseTable, StatusCode, StatusError

pytestmark = pytest.mark.gpu


def zipf_keys(n, vocab, s, seed):
    rng = np.random.default_rng(seed)
    k = rng.zipf(s, size=n).astype(np.int64) % vocab
    return torch.from_numpy(k * 2654435761 % (1 << 40))


def pair(dim, opt, n_shards=4, sync=False, **kw):
    g = SparseTable(dim, opt, kw or None, n_shards=n_shards, sync=sync, device="cuda", capacity=1 << 16,
                    max_keys=1 << 16)
    c = SparseTable(dim, opt, kw or None, n_shards=n_shards, sync=sync, device="cpu")
    return g, c


@pytest.mark.parametrize("dim", [16, 64, 128, 256])
def test_pull_matches_oracle_bitwise(dim):
    g, c = pair(dim, "adagrad", lr=0.05, init_accumulator=0.1)
    keys = zipf_keys(20000, 5000, 1.1, 0)
    a = g.pull(keys.cuda())
    g.check()
    b = c.pull(keys)
    assert torch.equal(a.cpu(), b)
    assert g.size() == c.size()
    assert g.engine.last_unique(0) == len(set(keys.tolist()))
    # second pull hits existing rows
    a2 = g.pull(keys.cuda())
    g.check()
    assert torch.equal(a2, a)


@pytest.mark.parametrize("opt,kw", [("sgd", dict(lr=0.1)), ("adagrad", dict(lr=0.05, init_accumulator=0.1)),
                                    ("ftrl", dict(alpha=0.05, beta=1.0, l1=0.001, l2=0.01)),
                                    ("adam", dict(lr=0.01)), ("sum", {})])
def test_push_unique_keys_bitwise(opt, kw):
    g, c = pair(32, opt, **kw)
    keys = torch.from_numpy(np.random.default_rng(1).permutation(1 << 20)[:8192].astype(np.int64))
    for step in range(3):
        grads = torch.randn(8192, 32, generator=torch.Generator().manual_seed(step)) * 1e-2
        g.pull(keys.cuda())
        g.push(grads.cuda())
        c.pull(keys)
        c.push(grads)
    g.check()
    a, fa = g.get_rows(keys.cuda(), emb_only=False)
    b, fb = c.get_rows(keys, emb_only=False)
    assert fa.all() and fb.all()
    assert torch.equal(a.cpu(), b)


def test_push_with_duplicates_close_to_oracle():
    g, c = pair(64, "adagrad", lr=0.05, init_accumulator=0.1)
    for step in range(4):
        keys = zipf_keys(30000, 4000, 1.05, step)
        grads = torch.randn(30000, 64, generator=torch.Generator().manual_seed(step)) * 1e-3
        g.pull(keys.cuda())
        g.push(grads.cuda())
        c.pull(keys)
        c.push(grads)
    g.check()
    uk = torch.unique(keys)
    a, _ = g.get_rows(uk.cuda(), emb_only=False)
    b, _ = c.get_rows(uk, emb_only=False)
    assert torch.allclose(a.cpu(), b, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("opt,kw", [("adagrad", dict(lr=0.05, init_accumulator=0.1)), ("ftrl", dict(alpha=0.05, beta=1.0, l1=0.001, l2=0.01))])
def test_deterministic_push_with_duplicates_is_bitwise_the_oracle(opt, kw):
    """In reproducible mode the duplicates of a batch are summed in a fixed order that depends on the batch alone
    (position order, in blocks of 64: tests/blocked_sum.py restates it on the host), as the reference's client-side
    merge makes the result a function of the request (pico-ps/operator/SparsePushOperator.h:130-146): the tables
    agree bit for bit with a host table that is given those sums, also for a batch whose head key repeats thousands
    of times."""
    from blocked_sum import blocked_segment_sum
    g, c = pair(64, opt, **kw)
    g.set_deterministic(True)
    for step in range(4):
        keys = zipf_keys(30000, 4000, 1.05, step)
        grads = torch.randn(30000, 64, generator=torch.Generator().manual_seed(step)) * 1e-3
        g.pull(keys.cuda())
        g.push(grads.cuda())
        c.pull(keys)
        uk_, agg_ = blocked_segment_sum(keys.numpy(), grads.numpy())
        c.push(torch.from_numpy(agg_), keys=torch.from_numpy(uk_))
    g.check()
    uk = torch.unique(torch.cat([zipf_keys(30000, 4000, 1.05, s_) for s_ in range(4)]))
    a, fa = g.get_rows(uk.cuda(), emb_only=False)
    b, fb = c.get_rows(uk, emb_only=False)
    assert fa.all() and fb.all() and torch.equal(a.cpu(), b)


def test_push_keeps_the_replica_exact_without_a_sync():
    """Replication inside the fused push (pico-ps/operator/SparsePushOperator.h:161-168: a push reaches every holder
    of a shard): the owner forwards key + folded gradient of every row it updates, the holder of the mirror applies
    the same step. After any number of pushes the mirror rows equal the primary rows bit for bit, with no sync in
    between, and a lost table is rebuilt from the mirror exactly. One GPU: the rank is its own partner."""
    from parameter_server_b200.parallel.migrate import ReplicaSet
    t = SparseTable(32, "adagrad", dict(lr=0.05, init_accumulator=0.1), device="cuda", capacity=1 << 15, max_keys=1 << 14,
                    replicate=True)
    rs = ReplicaSet(t, in_push=True)
    seen = []
    for step in range(5):
        keys = zipf_keys(12000, 3000 + 500 * step, 1.05, step).cuda()
        t.pull(keys)
        t.push(torch.randn(12000, 32, device="cuda") * 1e-2)
        seen.append(keys)
    t.check()
    uk = torch.unique(torch.cat(seen))
    a, fa = t.get_rows(uk, emb_only=False)
    b, fb = rs.mirror.get_rows(uk, emb_only=False)
    assert fa.all() and fb.all() and torch.equal(a, b)
    assert rs.mirror.size() == t.size() == uk.numel()
    # sync pushes append nothing but keep the hand-shake going; the next plain push still lands in the mirror
    # the table is lost between two steps; no sync() was ever called
    t.clear()
    assert t.size() == 0
    assert rs.restore(0) == uk.numel()
    c, fc = t.get_rows(uk, emb_only=False)
    assert fc.all() and torch.equal(c, a)
    # training goes on and the mirror keeps up
    t.pull(seen[0]); t.push(torch.ones(12000, 32, device="cuda") * 1e-2); t.check()
    u0 = torch.unique(seen[0])
    a, _ = t.get_rows(u0, emb_only=False)
    b, _ = rs.mirror.get_rows(u0, emb_only=False)
    assert torch.equal(a, b)


def test_pooling_and_mean_backward():
    g, c = pair(16, "sgd", lr=1.0)
    keys = zipf_keys(4096 * 4, 3000, 1.1, 3)
    for mean in (False, True):
        a = g.pull(keys.cuda(), bag_size=4, mean=mean)
        b = c.pull(keys, bag_size=4, mean=mean)
        assert torch.allclose(a.cpu(), b, rtol=1e-4, atol=1e-6)  # duplicate sums use atomics
        grads = torch.randn(4096, 16) * 1e-2
        g.push(grads.cuda())
        c.push(grads)
    g.check()
    uk = torch.unique(keys)
    a, _ = g.get_rows(uk.cuda())
    b, _ = c.get_rows(uk)
    assert torch.allclose(a.cpu(), b, rtol=1e-4, atol=1e-6)


def test_sync_push_then_store():
    g, c = pair(16, "adagrad", sync=True, lr=0.05, init_accumulator=0.1)
    keys = torch.arange(0, 3000, dtype=torch.int64) * 7919
    w0 = g.pull(keys.cuda()).clone()
    for step in range(2):
        grads = torch.randn(3000, 16, generator=torch.Generator().manual_seed(step)) * 1e-2
        g.pull(keys.cuda()); g.push(grads.cuda(), sync=True)
        c.pull(keys); c.push(grads, sync=True)
    assert torch.equal(g.pull(keys.cuda()), w0)
    g.store(); c.store()
    g.check()
    a, _ = g.get_rows(keys.cuda(), emb_only=False)
    b, _ = c.get_rows(keys, emb_only=False)
    assert torch.equal(a.cpu(), b)


def test_read_only_pull_and_autograd_lookup():
    t = SparseTable(16, "sgd", dict(lr=0.5), device="cuda", capacity=1 << 12, max_keys=1 << 12)
    keys = torch.arange(100, device="cuda")
    r = t.pull(keys, insert=False)
    assert t.size() == 0
    exp = torch.tensor([[C.init_uniform(k, d, 0, 0.01) for d in range(16)] for k in range(100)])
    assert torch.equal(r.cpu(), exp)
    emb = t.lookup(keys)
    loss = (emb * 2.0).sum()
    loss.backward()
    t.check()
    after, found = t.get_rows(keys)
    assert found.all()
    assert torch.allclose(after.cpu(), exp - 0.5 * 2.0)


def test_erase_export_set_rows_clear():
    g, c = pair(32, "adagrad", n_shards=3, lr=0.05, init_accumulator=0.1)
    keys = torch.arange(5000, dtype=torch.int64) * 104729
    g.pull(keys.cuda()); g.push(torch.ones(5000, 32).cuda() * 0.01)
    g.check()
    assert g.erase_keys(keys[::2].cuda()) == 2500
    assert g.size() == 2500
    ks, rs = [], []
    for k, r in g.export(batch=4096):
        ks.append(k); rs.append(r)
    ks, rs = torch.cat(ks), torch.cat(rs)
    assert sorted(ks.tolist()) == sorted(keys[1::2].tolist())
    per_shard = sum(k.numel() for s in range(3) for k, _ in g.export(shard=s))
    assert per_shard == 2500
    g2 = SparseTable(32, "adagrad", n_shards=5, device="cuda", capacity=1 << 14, max_keys=1 << 14)
    g2.set_rows(ks, rs)
    a, fa = g.get_rows(ks, emb_only=False)
    b, fb = g2.get_rows(ks, emb_only=False)
    assert fa.all() and fb.all() and torch.equal(a, b)
    # erased rows are recycled by later inserts
    g.pull(keys.cuda()); g.check()
    assert g.size() == 5000
    g.clear()
    assert g.size() == 0


def test_row_pool_limit_reports_oom_once_and_the_engine_keeps_working():
    """Memory pressure is not fatal: the call that met it runs to its end (scratch emptied, epoch advanced), the
    status is reported once, and later calls need no reset (pico-ps/operator/SparsePullOperator.h:195-199: pulls
    answer OUT_OF_MEMORY while items are parked, the server stays up)."""
    t = SparseTable(64, "adagrad", device="cuda", capacity=1 << 14, max_keys=1 << 13, max_rows=4096, slab_shift=12)
    first = t.pull(torch.arange(3000, device="cuda")); t.check()
    t.pull(torch.arange(3000, 8000, device="cuda"))
    st = t.status()
    assert st.code() == StatusCode.OUT_OF_MEMORY
    assert not t.table.healthy()
    assert t.status().ok()                      # reported once
    # no reset: read-only pulls keep answering and existing rows are intact
    for _ in range(3):
        r = t.pull(torch.arange(3000, device="cuda"), insert=False)
        t.check()
        assert torch.equal(r, first)
    # a key that found no row reads as its initial value and a push to it is dropped with OUT_OF_MEMORY again
    t.pull(torch.arange(7990, 8000, device="cuda"))
    t.push(torch.ones(10, 64, device="cuda"))
    assert t.status().code() == StatusCode.OUT_OF_MEMORY
    r = t.pull(torch.arange(10, device="cuda"), insert=False); t.check()
    assert torch.equal(r, first[:10])


def test_reserved_keys_are_refused_and_reset_rearms():
    t = SparseTable(16, "sgd", dict(lr=0.1), device="cuda", capacity=1 << 12, max_keys=1 << 10)
    good = torch.arange(100, device="cuda")
    want = t.pull(good); t.check()
    for reserved in (-(1 << 63), -(1 << 63) + 1):
        bad = good.clone()
        bad[7] = reserved
        t.pull(bad)
        st = t.status()
        assert st.code() == StatusCode.ERROR and "reserved" in st.msg()
        with pytest.raises(StatusError):        # a fatal status makes the engine refuse launches until reset()
            t.pull(good)
        t.reset()
        assert torch.equal(t.pull(good), want)
        t.check()
    assert t.size() == 100


def test_push_checks_the_gradient_row_count_and_an_unprepared_plan():
    t = SparseTable(16, "sum", device="cuda", capacity=1 << 12, max_keys=1 << 10)
    keys = torch.tensor([1, 2, 2, 3, 3, 3], device="cuda")
    t.pull(keys)
    with pytest.raises(StatusError):
        t.push(torch.ones(5, 16, device="cuda"))          # one row short: would read past the buffer
    with pytest.raises(StatusError):
        t.push(torch.ones(7, 16, device="cuda"))
    t.check()
    base = t.pull(keys, for_push=False).clone()           # the plan did not zero the aggregation rows ...
    t.push(torch.ones(6, 16, device="cuda"))              # ... so the push does it
    t.check()
    after = t.pull(keys, insert=False, for_push=False); t.check()
    assert torch.allclose(after - base, torch.tensor([1., 2., 2., 3., 3., 3.], device="cuda")[:, None].expand(6, 16), atol=1e-6)


@pytest.mark.parametrize("dim,bag", [(128, 1), (64, 1), (32, 4)])
def test_pull_in_bf16_is_the_fp32_pull_rounded_once(dim, bag):
    t = SparseTable(dim, "adagrad", dict(lr=0.05, init_accumulator=0.1), device="cuda", capacity=1 << 15, max_keys=1 << 14)
    keys = zipf_keys(8192, 3000, 1.1, 4).cuda()
    full = t.pull(keys, bag_size=bag, mean=bag > 1); t.check()
    half = t.pull(keys, bag_size=bag, mean=bag > 1, out_dtype=torch.bfloat16); t.check()
    assert half.dtype == torch.bfloat16 and torch.equal(half, full.to(torch.bfloat16))
    # the plan of a bf16 pull serves the push like any other
    t.push(torch.ones(8192 // bag, dim, device="cuda") * 1e-2); t.check()


def test_bounded_cta_budget_gives_the_same_results():
    g, c = pair(32, "adagrad", lr=0.05, init_accumulator=0.1)
    g.set_sm_budget(37, 50)
    assert g.engine.pull_blocks() <= 148 and g.engine.push_blocks() <= 148
    keys = torch.from_numpy(np.random.default_rng(3).permutation(1 << 20)[:20000].astype(np.int64))
    for step in range(3):
        grads = torch.randn(20000, 32, generator=torch.Generator().manual_seed(step)) * 1e-2
        a = g.pull(keys.cuda()); g.push(grads.cuda())
        b = c.pull(keys); c.push(grads)
        assert torch.equal(a.cpu(), b)
    g.check()
    a, _ = g.get_rows(keys.cuda(), emb_only=False)
    b, _ = c.get_rows(keys, emb_only=False)
    assert torch.equal(a.cpu(), b)


def test_sync_push_erase_reinsert_store_matches_oracle():
    """A row erased between sync_push and store leaves a stale entry in the touched list; when the row is recycled
    and touched again it must be folded exactly once."""
    g, c = pair(16, "ftrl", sync=True, alpha=0.05, beta=1.0, l1=0.001, l2=0.01)
    a_keys, b_keys = torch.arange(0, 512), torch.arange(512, 1024)
    for t_ in (g, c):
        dev = "cuda" if t_ is g else "cpu"
        gr = torch.ones(512, 16, device=dev) * 0.25
        t_.pull(a_keys.to(dev)); t_.push(gr, sync=True)
        assert t_.erase_keys(a_keys[:256].to(dev)) == 256
        t_.pull(b_keys.to(dev)); t_.push(gr * 2, sync=True)        # recycles the erased rows
        t_.pull(a_keys[:256].to(dev)); t_.push(gr[:256] * 3, sync=True)
        t_.store()
    g.check()
    allk = torch.arange(0, 1024)
    a, fa = g.get_rows(allk.cuda(), emb_only=False)
    b, fb = c.get_rows(allk, emb_only=False)
    assert fa.all() and fb.all() and torch.equal(a.cpu(), b)


def test_index_grows_between_replays_of_a_captured_step():
    """A job that keeps meeting new keys outgrows the index it started with. The host hook that runs before every
    launch (and before every replay of a captured step) doubles the index when its load would pass one half; the
    captured kernels read the table through a view in device memory, so they follow the growth."""
    g, c = pair(16, "adagrad", lr=0.05, init_accumulator=0.1)
    t = SparseTable(16, "adagrad", dict(lr=0.05, init_accumulator=0.1), n_shards=4, device="cuda", capacity=2048, max_keys=4096)
    assert t.table.index_capacity() == 4096
    keys_buf = torch.zeros(4096, dtype=torch.int64, device="cuda")
    grads = torch.full((4096, 16), 1e-2, device="cuda")
    out = torch.empty(4096, 16, device="cuda")
    t.opt.step_from_epoch = 1
    for _ in range(2):                                   # eager warm-up on the first keys
        keys_buf.copy_(torch.arange(4096, device="cuda") * 31)
        t.reserve(4096); t.pull(keys_buf, out=out); t.push(grads)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    t.reserve(4 * 4096)
    with torch.cuda.graph(graph):
        t.pull(keys_buf, out=out); t.push(grads)
    seen = [torch.arange(4096) * 31] * 2
    for step in range(40):                               # 40 x 4096 new keys through a graph captured at 4096 slots
        k = torch.arange(4096) * 31 + (step + 1) * 1000003
        keys_buf.copy_(k.cuda())
        t.reserve(4096)
        graph.replay()
        seen.append(k)
    t.check()
    assert t.table.grow_count() >= 3 and t.table.index_capacity() >= 2 * t.size()
    for k in seen:
        c.pull(k); c.push(grads.cpu())
    allk = torch.unique(torch.cat(seen))
    assert t.size() == allk.numel() == c.size()
    a, fa = t.get_rows(allk.cuda(), emb_only=False)
    b, fb = c.get_rows(allk, emb_only=False)
    assert fa.all() and fb.all() and torch.equal(a.cpu(), b)


def test_large_batch_1m_keys():
    g = SparseTable(64, "adagrad", dict(lr=0.05, init_accumulator=0.1), device="cuda", capacity=1 << 21,
                    max_keys=1 << 20)
    keys = zipf_keys(1 << 20, 1 << 22, 1.05, 9).cuda()
    out = g.pull(keys)
    g.push(torch.full((1 << 20, 64), 1e-3, device="cuda"))
    g.check()
    nu = g.engine.last_unique(0)
    assert nu == torch.unique(keys).numel() == g.size()
    assert torch.isfinite(out).all()


def test_cold_tier_spill_fetch_and_persistence(tmp_path):
    t = SparseTable(32, "adagrad", dict(lr=0.05, init_accumulator=0.1), device="cuda", capacity=1 << 15, max_keys=1 << 14)
    t.enable_cold_tier(1 << 14, window=4096)
    hot, cold = torch.arange(0, 4000, device="cuda"), torch.arange(4000, 10000, device="cuda")
    t.pull(torch.cat([hot, cold]))
    for _ in range(3):                      # only the hot keys keep receiving gradient
        t.pull(hot); t.push(torch.ones(4000, 32, device="cuda"))
    t.check()
    full, _ = t.get_rows(torch.cat([hot, cold]), emb_only=False)
    n = t.spill_cold(section=1, threshold=0.5)          # Adagrad accumulator stayed at 0.1 for the cold keys
    assert n == 6000 and t.size() == 4000 and t.cold.size() == 6000
    # persistence with the layout identity check
    img = str(tmp_path / "cold.img")
    assert t.cold.save(img, "uuid-A").ok()
    t2 = SparseTable(32, "adagrad", dict(lr=0.05, init_accumulator=0.1), device="cuda", capacity=1 << 15, max_keys=1 << 14)
    t2.enable_cold_tier(1 << 14)
    assert t2.cold.load(img, "uuid-B").code() == StatusCode.INVALID_ID
    assert t2.cold.load(img, "uuid-A").ok() and t2.cold.size() == 6000
    # the next batch touches some cold keys: fetch them back first, nothing was lost (slots included)
    batch = torch.cat([hot[:100], cold[:500]]).cpu()
    assert t.prefetch_cold(batch) == 500 and t.cold.size() == 5500 and t.size() == 4500
    rows, found = t.get_rows(batch.cuda(), emb_only=False)
    assert found.all()
    assert torch.equal(rows, torch.cat([full[:100], full[4000:4500]]))
    assert t.spill_keys(hot[:10]) == 10 and t.size() == 4490
    # asynchronous prefetch of the next batch's cold rows: staged off the critical path, inserted between steps
    nxt = torch.cat([cold[1000:1300], hot[:10]]).cpu()
    t.prefetch_cold_async(nxt)
    t.pull(hot[100:200]); t.push(torch.zeros(100, 32, device="cuda"))     # the current step keeps running
    assert t.commit_prefetch() == 310 and t.size() == 4800
    rows, found = t.get_rows(cold[1000:1300], emb_only=False)
    assert found.all() and torch.equal(rows, full[5000:5300])
    t.check()


def test_collective_dump_load_rehash_and_rpc_codec(tmp_path):
    from parameter_server_b200.parallel import checkpoint
    t = SparseTable(16, "ftrl", dict(lr=0.05), device="cuda", n_shards=4, capacity=1 << 14, max_keys=1 << 13)
    keys = torch.randint(0, 1 << 40, (5000,), device="cuda")
    t.pull(keys); t.push(torch.randn(5000, 16, device="cuda") * 1e-2); t.check()
    uniq = torch.unique(keys)
    want, _ = t.get_rows(uniq, emb_only=False)
    assert checkpoint.dump(t, str(tmp_path / "d"), file_number=3) == t.size()
    assert sorted(os.listdir(tmp_path / "d")) == ["model_0_0", "model_0_1", "model_0_2"]
    t2 = SparseTable(16, "ftrl", dict(lr=0.05), device="cuda", n_shards=7, capacity=1 << 14, max_keys=1 << 13)
    assert checkpoint.load(t2, str(tmp_path / "d")) == t.size()
    got, found = t2.get_rows(uniq, emb_only=False)
    assert found.all() and torch.equal(got, want)
    # the files are the RPC path's binary codec: a host table behind the service layer's reader gets the same rows
    raw = open(tmp_path / "d" / "model_0_0", "rb").read()
    assert raw[:4] == b"PSB1" and int.from_bytes(raw[4:8], "little") == t.table.stride()
    assert (len(raw) - 8) % (8 + 4 * t.table.stride()) == 0


def test_cold_tier_policy_keeps_hbm_rows_under_budget_and_loses_nothing():
    from parameter_server_b200.ops.cold_policy import ColdTierPolicy
    t = SparseTable(16, "adagrad", dict(lr=0.05, init_accumulator=0.1), device="cuda", capacity=1 << 15, max_keys=1 << 12)
    ref = SparseTable(16, "adagrad", dict(lr=0.05, init_accumulator=0.1), device="cuda", capacity=1 << 15, max_keys=1 << 12)
    pol = ColdTierPolicy(t, hbm_budget_rows=3000, cold_capacity_rows=1 << 14, interval=5, headroom=0.2)
    g = torch.Generator().manual_seed(0)
    batches = [torch.randint(0, 8000, (2048,), generator=g) for _ in range(40)]
    over = []
    for i, kh in enumerate(batches):
        k = kh.cuda()
        out = pol.pull(k, kh)
        grads = torch.ones(2048, 16, device="cuda") * 0.01 * (1 + (k % 3)).float()[:, None]
        t.push(grads)
        want = ref.pull(k); ref.push(grads)
        assert torch.equal(out, want), f"step {i}: a row came back different from the never-spilled table"
        pol.maybe_spill()
        over.append(t.size())
    t.check(); ref.check()
    assert pol.spilled_total > 0 and pol.fetched_total > 0
    assert t.size() + t.cold.size() == ref.size()
    # right after a spill the table is under its budget
    assert min(over[4::5]) <= 3000
    # staged prefetch one step ahead
    nxt = batches[0]
    pol.stage_next(nxt)
    out = pol.pull(nxt.cuda(), nxt)
    assert torch.equal(out, ref.pull(nxt.cuda()))
