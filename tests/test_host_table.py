"""CPU storage + oracle semantics (pull inserts, dedup, pre-aggregation, sync push + store, erase,
export), modelled on pico-ps/test/ps_service_test.cpp:77-239."""
import numpy as np
import pytest
import torch

from parameter_server_b200 import C, SparseTable, make_opt_config


def mk(dim=8, opt="sum", sync=False, n_shards=4, **kw):
    return SparseTable(dim, opt, kw or None, n_shards=n_shards, sync=sync, device="cpu")


def test_pull_inserts_and_is_deterministic():
    t = mk()
    keys = torch.tensor([5, 9, 5, 1 << 39, 9], dtype=torch.int64)
    a = t.pull(keys)
    assert t.size() == 3
    b = t.pull(keys)
    assert torch.equal(a, b)
    assert torch.equal(a[0], a[2]) and torch.equal(a[1], a[4])
    exp = np.array([C.init_uniform(5, d, 0, 0.01) for d in range(8)], dtype=np.float32)
    assert np.array_equal(a[0].numpy(), exp)


def test_read_only_pull_does_not_insert():
    t = SparseTable(8, "sum", n_shards=2, read_only=True, device="cpu")
    a = t.pull(torch.tensor([1, 2, 3]))
    assert t.size() == 0
    exp = np.array([C.init_uniform(2, d, 0, 0.01) for d in range(8)], dtype=np.float32)
    assert np.array_equal(a[1].numpy(), exp)


def test_push_preaggregates_duplicates_sum():
    t = mk(dim=4)
    keys = torch.tensor([7, 7, 8, 7])
    base = t.pull(keys).clone()
    g = torch.arange(16, dtype=torch.float32).reshape(4, 4)
    t.push(g)
    after = t.pull(torch.tensor([7, 8]))
    assert torch.allclose(after[0], base[0] + g[0] + g[1] + g[3])
    assert torch.allclose(after[1], base[2] + g[2])


def test_adagrad_matches_formula():
    t = mk(dim=4, opt="adagrad", lr=0.05, init_accumulator=0.1)
    k = torch.tensor([42])
    w0 = t.pull(k).clone()
    g = torch.tensor([[1e-3, -2e-3, 3e-3, 0.0]])
    t.push(g)
    w1 = t.pull(k)
    acc = 0.1 + g * g
    exp = w0 - 0.05 * g / (acc.sqrt() + 1e-10)
    assert torch.allclose(w1, exp, rtol=1e-6, atol=1e-9)
    rows, found = t.get_rows(k, emb_only=False)
    assert found[0] == 1 and torch.allclose(rows[0, 4:], acc[0])


def test_sync_push_is_buffered_until_store():
    t = mk(dim=4, opt="sgd", sync=True, lr=1.0)
    k = torch.tensor([1, 2])
    w0 = t.pull(k).clone()
    g = torch.ones(2, 4)
    t.push(g, sync=True)
    t.pull(k)
    t.push(g, sync=True)
    assert torch.equal(t.pull(k), w0)  # nothing applied yet
    t.store()
    assert torch.allclose(t.pull(k), w0 - 2.0)
    t.store()  # idempotent when nothing is pending
    assert torch.allclose(t.pull(k), w0 - 2.0)


def test_pooling_sum_and_mean():
    t = mk(dim=4)
    keys = torch.tensor([1, 2, 3, 3, 4, 5])
    rows = t.pull(keys)
    s = t.pull(keys, bag_size=3)
    m = t.pull(keys, bag_size=3, mean=True)
    assert torch.allclose(s[0], rows[:3].sum(0)) and torch.allclose(s[1], rows[3:].sum(0))
    assert torch.allclose(m, s / 3)


def test_erase_export_set_rows_round_trip():
    t = mk(dim=4, opt="adagrad", n_shards=3)
    keys = torch.arange(100, dtype=torch.int64)
    t.pull(keys)
    t.push(torch.randn(100, 4))
    assert t.erase_keys(torch.arange(0, 100, 2)) == 50
    assert t.size() == 50
    got = {}
    for k, r in t.export(batch=16):
        for kk, rr in zip(k.tolist(), r):
            got[kk] = rr.clone()
    assert sorted(got) == list(range(1, 100, 2))
    t2 = mk(dim=4, opt="adagrad", n_shards=5)  # different sharding: load rehashes
    ks = torch.tensor(sorted(got))
    t2.set_rows(ks, torch.stack([got[k] for k in sorted(got)]))
    a, fa = t.get_rows(ks, emb_only=False)
    b, fb = t2.get_rows(ks, emb_only=False)
    assert fa.all() and fb.all() and torch.equal(a, b)


def test_memory_limit_turns_into_oom_status():
    t = SparseTable(64, "adagrad", n_shards=1, device="cpu", memory_limit_bytes=64 * 1024)
    from parameter_server_b200 import StatusError, StatusCode
    with pytest.raises(StatusError) as ei:
        for i in range(100):
            t.pull(torch.arange(i * 100, (i + 1) * 100))
    assert ei.value.code == StatusCode.OUT_OF_MEMORY
    assert not t.table.healthy()


@pytest.mark.parametrize("opt,kw", [("sgd", dict(lr=0.1)), ("adagrad", dict(lr=0.05, init_accumulator=0.1)),
                                    ("ftrl", dict(alpha=0.05, beta=1.0, l1=0.001, l2=0.01)),
                                    ("adam", dict(lr=0.01))])
def test_optimizers_move_weights(opt, kw):
    t = mk(dim=4, opt=opt, **kw)
    k = torch.tensor([3])
    w0 = t.pull(k).clone()
    for _ in range(3):
        t.pull(k)
        t.push(torch.full((1, 4), 0.5))
    w1 = t.pull(k)
    assert torch.all(w1 < w0) or opt == "ftrl"
    assert torch.isfinite(w1).all()


def test_dropping_a_shard_takes_its_items_out_of_the_count():
    t = mk(n_shards=4)
    keys = torch.arange(400, dtype=torch.int64)
    t.pull(keys)
    assert t.size() == 400
    per_shard = {s: t.table.shard_size(s) for s in t.table.shard_list()}
    assert sum(per_shard.values()) == 400
    t.table.erase_shard(2)
    assert t.size() == 400 - per_shard[2] and 2 not in t.table.shard_list()
    assert t.memory_usage() >= 0
    t.table.create_shard(2)
    assert t.table.shard_size(2) == 0 and t.size() == 400 - per_shard[2]


def test_health_comes_back_when_there_is_room_again():
    from parameter_server_b200 import StatusError
    t = SparseTable(64, "adagrad", n_shards=1, device="cpu", memory_limit_bytes=64 * 1024)
    keys = []
    with pytest.raises(StatusError):
        for i in range(100):
            k = torch.arange(i * 20, (i + 1) * 20)
            t.pull(k)
            keys.append(k)
    assert not t.table.healthy()
    assert not t.table.check_healthy()                 # still no room: the monitor leaves the flag down
    assert t.erase_keys(torch.cat(keys)[:60]) == 60    # room again: 60 row slots on the free list
    assert t.table.check_healthy() and t.table.healthy()
    t.pull(torch.arange(10**6, 10**6 + 50))            # new rows fit into the freed slots
    assert t.table.healthy()
    # raising the limits is the other way back
    with pytest.raises(StatusError):
        for i in range(100):
            t.pull(torch.arange(2 * 10**6 + i * 50, 2 * 10**6 + (i + 1) * 50))
    assert not t.table.check_healthy()
    t.table.set_limits(1 << 20, 1 << 20)
    assert t.table.check_healthy()
    # and a table pushed over a limit that was lowered afterwards is marked without waiting for a failed insert
    t.table.set_limits(1024, 1024)
    assert not t.table.check_healthy() and not t.table.healthy()


def test_a_push_that_hits_the_memory_limit_is_applied_exactly_once():
    """A push is taken as a whole or refused as a whole: items that find no row when the limit is hit are parked (the
    reference's overflow list), the next requests are refused up front, and the parked items are applied when there
    is room again - so a client that retries after OUT_OF_MEMORY never counts a gradient twice."""
    from parameter_server_b200 import StatusError, StatusCode
    t = SparseTable(64, "sum", n_shards=2, device="cpu", memory_limit_bytes=64 * 1024, init_range=0.0)
    keys = torch.arange(1000)
    t._plan_keys = None
    ones = torch.ones(1000, 64)
    t.table.push(keys.numpy(), ones.numpy(), t.opt)               # accepted as a whole although only part fits
    placed, parked = t.size(), t.table.overflow_size()
    assert 0 < placed < 1000 and placed + parked == 1000 and not t.table.healthy()
    st = t.table.push(keys.numpy(), ones.numpy(), t.opt)          # refused before anything is applied
    assert st.code() == StatusCode.OUT_OF_MEMORY and t.table.overflow_size() == parked
    st, _ = t.table.pull(keys.numpy())                            # pulls of a shard with parked items say so
    assert st.code() == StatusCode.OUT_OF_MEMORY
    t.table.set_limits(1 << 22, 1 << 22)                          # room again: the monitor drains the list
    assert t.table.check_healthy() and t.table.overflow_size() == 0 and t.size() == 1000
    st = t.table.push(keys.numpy(), ones.numpy(), t.opt)          # the client's retry
    assert st.ok()
    rows, found = t.get_rows(keys)
    assert bool(found.all()) and torch.equal(rows, 2 * ones)      # every gradient exactly once


def test_expected_max_items_sizes_the_index_up_front():
    hc = C.HostTableConfig()
    hc.dim, hc.n_shards = 4, 2
    small = C.HostTable(hc)
    hc.expected_max_items = 100_000
    big = C.HostTable(hc)
    for t in (small, big):
        t.create_shard(0)
    buckets = lambda t: t.export_shard(0, 0, 1 << 30, False)[2]      # the scan cursor ends at the bucket count
    assert buckets(big) >= 2 * 50_000 and buckets(small) < 1024      # load factor <= 1/2 for the shard's share
    keys = np.arange(20_000, dtype=np.int64)
    before = buckets(big)
    big.create_shard(1)
    big.set_rows(keys, np.zeros((20_000, 4), np.float32), False)
    assert buckets(big) == before                                     # filling it did not rebuild the index


def test_grow_and_shrink_ratio_of_the_index():
    """`grow_ratio` is the load at which a shard's index doubles, `shrink_ratio` the load under which it is rebuilt
    smaller after keys were erased (the resizing parameters of the reference's storage configs)."""
    buckets = lambda t: t.export_shard(0, 0, 1 << 30, False)[2]
    n = 3000
    keys = np.arange(n, dtype=np.int64)
    sizes = {}
    for grow in (0.0, 0.25, 0.8, 2.0):
        hc = C.HostTableConfig()
        hc.dim, hc.n_shards = 4, 1
        hc.index_grow_ratio = grow
        t = C.HostTable(hc)
        t.create_shard(0)
        t.set_rows(keys, np.ones((n, 4), np.float32), True)
        sizes[grow] = buckets(t)
        load = n / buckets(t)
        assert load <= (min(max(grow, 0.25), 0.85) if grow else 0.5) + 1e-9
        rows, found = t.get_rows(keys, True)
        assert found.all() and np.all(rows[:, :4] == 1.0)
    assert sizes[0.25] > sizes[0.0] >= sizes[0.8] == sizes[2.0]       # 2.0 is clamped: open addressing needs room
    for shrink in (0.0, 0.2):
        hc = C.HostTableConfig()
        hc.dim, hc.n_shards = 4, 1
        hc.index_shrink_ratio = shrink
        t = C.HostTable(hc)
        t.create_shard(0)
        t.set_rows(keys, np.ones((n, 4), np.float32), True)
        full = buckets(t)
        assert t.erase_keys(keys[100:]) == n - 100
        if shrink:
            assert buckets(t) < full and 100 / buckets(t) <= 0.5
        else:
            assert buckets(t) == full
        rows, found = t.get_rows(keys, True)
        assert found[:100].all() and not found[100:].any()
        t.set_rows(keys, 2 * np.ones((n, 4), np.float32), True)      # grows back
        rows, found = t.get_rows(keys, True)
        assert found.all() and np.all(rows[:, :4] == 2.0) and t.size() == n


def test_layout_epoch_moves_exactly_when_bucket_cursors_lose_their_meaning():
    hc = C.HostTableConfig()
    hc.dim, hc.n_shards = 4, 1
    hc.expected_max_items = 1000
    hc.index_shrink_ratio = 0.2
    t = C.HostTable(hc)
    assert t.layout_epoch(0) == 0                                     # no such shard
    t.create_shard(0)
    e0 = t.layout_epoch(0)
    keys = np.arange(1000, dtype=np.int64)
    t.set_rows(keys, np.ones((1000, 4), np.float32), True)
    assert t.layout_epoch(0) == e0                                    # inserts into a table with room move nothing
    # a scan by cursor in two halves sees every key once while the epoch stands
    half = t.export_shard(0, 0, 1 << 30, False)[2] // 2
    k1, _, c, fin = t.export_shard(0, 0, half, False)
    k2, _, c, fin2 = t.export_shard(0, c, 1 << 30, False)
    assert not fin and fin2 and sorted(np.concatenate([k1, k2]).tolist()) == keys.tolist()
    t.set_rows(np.arange(1000, 5000, dtype=np.int64), np.ones((4000, 4), np.float32), True)
    e1 = t.layout_epoch(0)
    assert e1 != e0                                                   # growth rebuilt the index
    t.erase_keys(np.arange(100, 5000, dtype=np.int64))
    e2 = t.layout_epoch(0)
    assert e2 != e1                                                   # so did the shrink after the erase
    t.erase_shard(0)
    t.create_shard(0)
    assert t.layout_epoch(0) not in (e0, e1, e2)                      # a shard created anew is another shard


def test_health_does_not_flap_while_parked_items_find_no_room():
    """Rows freed in one shard do not help the parked items of another: the table drains what it can at every
    re-evaluation and stays unhealthy until the last parked item has a row."""
    hc = C.HostTableConfig()
    hc.dim, hc.n_shards = 64, 2
    hc.soft_limit_bytes = hc.hard_limit_bytes = 64 * 1024
    t = C.HostTable(hc)
    t.create_shard(0)
    t.create_shard(1)
    opt = C.OptConfig()
    keys = np.arange(300, dtype=np.int64)
    shard = C.sparse_shards_of(keys, 2, [])
    for i in range(3):
        st = t.push(keys[i * 100:(i + 1) * 100], np.ones((100, 64), np.float32), opt)
        if not t.healthy():
            break
    assert st.ok() and not t.healthy() and t.overflow_size() > 0          # the push that hit the limit was taken whole
    parked_before = t.overflow_size()
    # the shard whose row pool could not double holds the parked items; free rows in the OTHER shard only
    full = 0 if t.shard_size(0) < t.shard_size(1) else 1
    have = keys[:(i + 1) * 100]
    rows, found = t.get_rows(have, True)
    lone = have[(found == 1) & (shard[:len(have)] == 1 - full)]
    assert t.erase_keys(lone[:40]) == 40
    for _ in range(3):
        assert not t.check_healthy()                                       # no healthy moment in between
        assert t.overflow_size() == parked_before                          # those rows are of no use to the full shard
    # now the full shard makes room as well
    mine = have[(found == 1) & (shard[:len(have)] == full)]
    assert t.erase_keys(mine[: parked_before + 5]) == parked_before + 5
    assert t.check_healthy() and t.overflow_size() == 0
    assert t.push(keys[:10], np.ones((10, 64), np.float32), opt).ok()


def test_reserved_keys_are_refused_by_the_host_table_and_the_collective_cpu_path():
    """INT64_MIN and INT64_MIN + 1 mark empty and erased buckets: pull / push / set_rows refuse them with a status,
    reads report them absent; nothing is inserted."""
    from parameter_server_b200 import SparseTable
    from parameter_server_b200.utils.status import StatusError
    t = SparseTable(8, "adagrad", dict(lr=0.1), device="cpu", group="none")
    t.pull(torch.arange(10))
    for k in (-2 ** 63, -2 ** 63 + 1):
        for call in (lambda: t.pull(torch.tensor([5, k])), lambda: t.pull(torch.tensor([k]), insert=False),
                     lambda: t.push(torch.ones(2, 8), torch.tensor([5, k])),
                     lambda: t.set_rows(torch.tensor([k]), torch.ones(1, 16))):
            with pytest.raises(StatusError) as e:
                call()
            assert "reserved" in str(e.value)
        assert t.get_rows(torch.tensor([k]))[1].tolist() == [0] and t.erase_keys(torch.tensor([k])) == 0
    assert t.size() == 10
