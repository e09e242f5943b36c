"""Property tests of the host storage / oracle against an independent numpy model, and of the codecs.

The CPU oracle (`HostTable`) is what every GPU kernel is compared with bit for bit, so it is itself
checked here against the textbook formulas written out in numpy (float32 arithmetic, the same order of
operations), over random sequences of pulls, pushes with duplicates, sync pushes + store, erases and
set_rows. Modelled on the per-key invariants that the reference asserts inside its test operators
(pico-ps/test/TestOps.h:87-118)."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from parameter_server_b200 import C, SparseTable

DIM = 4
F = np.float32


class Model:
    """key -> [w | slots] in float32, updated with the formulas of each optimizer."""

    def __init__(self, opt, kw):
        self.opt, self.kw, self.rows = opt, kw, {}

    def _init(self, key):
        w = np.array([C.init_uniform(int(key), d, 0, 0.01) for d in range(DIM)], dtype=F)
        if self.opt == "adagrad":
            return [w, np.full(DIM, self.kw.get("init_accumulator", 0.1), dtype=F)]
        if self.opt in ("sgd", "sum"):
            return [w]
        raise NotImplementedError(self.opt)

    def pull(self, keys):
        out = []
        for k in keys:
            if k not in self.rows:
                self.rows[k] = self._init(k)
            out.append(self.rows[k][0].copy())
        return np.stack(out)

    def push(self, keys, grads):
        agg = {}
        for k, g in zip(keys, grads):          # client-side pre-aggregation in batch order
            agg[k] = agg.get(k, np.zeros(DIM, dtype=F)) + g.astype(F)
        for k, g in agg.items():
            if k not in self.rows:
                self.rows[k] = self._init(k)
            r = self.rows[k]
            if self.opt == "sum":
                r[0] = (r[0] + g).astype(F)
            elif self.opt == "sgd":
                r[0] = (r[0] - F(self.kw["lr"]) * g).astype(F)
            elif self.opt == "adagrad":
                r[1] = (r[1] + g * g).astype(F)
                r[0] = (r[0] - F(self.kw["lr"]) * g / (np.sqrt(r[1]) + F(1e-10))).astype(F)

    def erase(self, keys):
        for k in set(keys):
            self.rows.pop(k, None)


ops = st.lists(st.tuples(st.sampled_from(["pull", "push", "erase"]),
                         st.lists(st.integers(min_value=0, max_value=40), min_size=1, max_size=24),
                         st.integers(min_value=0, max_value=2 ** 31 - 1)), min_size=1, max_size=25)


@pytest.mark.parametrize("opt,kw,exact", [("sum", {}, True), ("sgd", {"lr": 0.5}, True),
                                          ("adagrad", {"lr": 0.05, "init_accumulator": 0.1}, False)])
@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(ops=ops, n_shards=st.integers(min_value=1, max_value=7))
def test_host_table_follows_the_textbook_model(opt, kw, exact, ops, n_shards):
    t = SparseTable(DIM, opt, kw or None, n_shards=n_shards, device="cpu")
    m = Model(opt, kw)
    for kind, keys, seed in ops:
        k = torch.tensor(keys, dtype=torch.int64)
        if kind == "pull":
            got = t.pull(k).numpy()
            want = m.pull(keys)
            assert np.array_equal(got, want) if exact else np.allclose(got, want, rtol=1e-6, atol=1e-9)
        elif kind == "push":
            g = np.random.default_rng(seed).standard_normal((len(keys), DIM)).astype(F) * F(0.01)
            t.pull(k)                       # the push plan comes from the last pull
            m.pull(keys)
            t.push(torch.from_numpy(g))
            m.push(keys, g)
        else:
            t.erase_keys(k)
            m.erase(keys)
        assert t.size() == len(m.rows)
    # final state, slots included
    if m.rows:
        ks = sorted(m.rows)
        rows, found = t.get_rows(torch.tensor(ks, dtype=torch.int64), emb_only=False)
        assert found.all()
        want = np.stack([np.concatenate(m.rows[k]) for k in ks])
        assert np.array_equal(rows.numpy(), want) if exact else np.allclose(rows.numpy(), want, rtol=1e-6, atol=1e-9)


@settings(max_examples=80, deadline=None)
@given(keys=st.lists(st.integers(min_value=-(2 ** 62), max_value=2 ** 62), min_size=1, max_size=64, unique=True),
       n_old=st.integers(min_value=1, max_value=64), grow=st.integers(min_value=1, max_value=8))
def test_jump_hash_moves_keys_only_to_new_shards(keys, n_old, grow):
    """Consistent hashing: growing the shard count from n to n + g never moves a key between OLD shards."""
    for k in keys:
        a, b = C.sparse_shard_of(k, n_old), C.sparse_shard_of(k, n_old + grow)
        assert 0 <= a < n_old and 0 <= b < n_old + grow
        assert b == a or b >= n_old


@settings(max_examples=100, deadline=None)
@given(i=st.integers(min_value=-(2 ** 63), max_value=2 ** 63 - 1), d=st.floats(allow_nan=False),
       s=st.text(max_size=40), v=st.lists(st.integers(min_value=-(2 ** 31), max_value=2 ** 31 - 1), max_size=20),
       vs=st.lists(st.text(max_size=12), max_size=6))
def test_archive_round_trip(i, d, s, v, vs):
    i2, d2, s2, v2, vs2, code, msg, exhausted, _ = C.archive_round_trip(i, d, s, v, vs)
    assert (i2, s2, list(v2), list(vs2)) == (i, s, v, vs) and d2 == d
    assert code == 3 and msg == "full" and exhausted            # the Status that follows survives too


@settings(max_examples=40, deadline=None)
@given(data=st.binary(max_size=4096), algo=st.sampled_from(["", "zstd", "lz4", "snappy"]))
def test_compression_round_trip(data, algo):
    stt, back, _ = C.compress_round_trip(algo, data)
    assert stt.ok() and back == data


json_values = st.recursive(st.none() | st.booleans() | st.integers(min_value=-(2 ** 53), max_value=2 ** 53) |
                           st.floats(allow_nan=False, allow_infinity=False, width=32) | st.text(max_size=12),
                           lambda children: st.lists(children, max_size=4) | st.dictionaries(st.text(max_size=6), children, max_size=4),
                           max_leaves=20)


@settings(max_examples=150, deadline=None)
@given(text=st.text(max_size=200) | json_values.map(lambda v: __import__("json").dumps(v)))
def test_descriptor_parser_never_crashes_and_rejects_what_is_not_a_context(text):
    from parameter_server_b200 import service as S
    td = S.TableDescriptor()
    before = td.to_json_str()
    ok = td.from_json_str(text)
    if not ok:
        assert td.to_json_str() == before                  # a rejected input leaves the descriptor alone


def test_deeply_nested_json_is_refused_not_followed():
    from parameter_server_b200 import service as S
    td = S.TableDescriptor()
    for n in (200, 100000, 2000000):
        assert td.from_json_str("[" * n + "]" * n) is False
        assert td.from_json_str('{"a":' * n + "1" + "}" * n) is False
    # a real context still round-trips
    good = td.to_json_str()
    td2 = S.TableDescriptor()
    assert td2.from_json_str(good) and td2.to_json_str() == good


@settings(max_examples=60, deadline=None)
@given(data=st.binary(min_size=1, max_size=2048), algo=st.sampled_from(["zstd", "lz4"]), flips=st.lists(st.integers(0, 4095), min_size=1, max_size=8),
       cut=st.integers(0, 64))
def test_damaged_compressed_blocks_are_refused_not_followed(data, algo, flips, cut):
    """Bit flips, truncation and hostile size headers in a compressed block end in an error status (or, by chance,
    in other data): never in a crash or an absurd allocation."""
    stt, packed = C.compress_only(algo, data)
    assert stt.ok()
    b = bytearray(packed)
    for f in flips:
        b[f % len(b)] ^= 1 << (f % 8)
    b = bytes(b[: max(1, len(b) - cut)])
    stt, _ = C.decompress_only(algo, b)                      # any status, but it returns
    hostile = (2 ** 62).to_bytes(8, "little") + packed[8:]
    assert not C.decompress_only(algo, hostile)[0].ok()


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(batches=st.lists(st.lists(st.integers(min_value=0, max_value=300), min_size=1, max_size=40), min_size=1, max_size=25),
       period=st.integers(min_value=2, max_value=9), n_shards=st.integers(min_value=1, max_value=4),
       opt=st.sampled_from(["sum", "adagrad"]))
def test_pushes_are_applied_exactly_once_whatever_inserts_fail(batches, period, n_shards, opt):
    """Allocation failures injected into the inserts of new keys (every `period`-th one): a pushing client that does
    what the handlers do - send again after OUT_OF_MEMORY, once the monitor saw room - ends with the same table as a
    client of a table where nothing ever failed. Items are parked, never lost, never applied twice."""
    kw = dict(lr=0.1, init_accumulator=0.1) if opt == "adagrad" else None
    flaky = SparseTable(DIM, opt, kw, n_shards=n_shards, device="cpu", init_range=0.0)
    calm = SparseTable(DIM, opt, kw, n_shards=n_shards, device="cpu", init_range=0.0)
    flaky.table.inject_insert_failures(period)
    for i, b in enumerate(batches):
        keys = np.asarray(b, dtype=np.int64)
        grads = np.full((len(b), DIM), 1.0 + i, dtype=F)
        assert calm.table.push(keys, grads, calm.opt).ok()
        for attempt in range(200):
            status = flaky.table.push(keys, grads, flaky.opt)
            if status.ok():
                break
            assert status.code() == C.StatusCode.OUT_OF_MEMORY
            flaky.table.check_healthy()            # the monitor: there is room (no limit), parked items are retried
        else:
            raise AssertionError("the push was never let in")
    flaky.table.inject_insert_failures(0)
    for _ in range(3):
        flaky.table.check_healthy()
    assert flaky.table.overflow_size() == 0 and flaky.table.healthy()
    assert flaky.size() == calm.size()
    keys = torch.arange(0, 301)
    got, found_a = flaky.get_rows(keys, emb_only=False)
    want, found_b = calm.get_rows(keys, emb_only=False)
    assert torch.equal(found_a, found_b)
    if opt == "sum":
        assert torch.equal(got, want)
    else:
        # parked gradients of one key are applied after later pushes of that key were refused and sent again, never
        # interleaved differently from the order of acceptance; Adagrad is order-sensitive only in rounding
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)


@settings(max_examples=150, deadline=None)
@given(data=st.binary(max_size=3000))
def test_base64_and_config_blobs_round_trip(data):
    import base64
    import json
    text = C.base64_encode(data)
    assert text == base64.b64encode(data).decode()              # the standard alphabet and padding
    assert C.base64_decode(text) == data
    conf = C.add_base64_config(json.dumps({"dim": 8}), "blob", data)
    assert json.loads(conf)["dim"] == 8 and isinstance(json.loads(conf)["blob"], str)
    status, back = C.get_base64_config(conf, "blob")
    assert status.ok() and back == data
    assert C.byte2str(data) == data.hex()


@settings(max_examples=150, deadline=None)
@given(text=st.text(alphabet="ABCDabcd0189+/=_ \n", max_size=40))
def test_base64_decoder_refuses_what_is_not_base64(text):
    import base64
    import binascii
    got = C.base64_decode(text)
    try:
        want = base64.b64decode(text, validate=True) if len(text) % 4 == 0 else None
    except binascii.Error:
        want = None
    if want is None:
        assert got is None
    else:
        assert got == want
    assert not C.get_base64_config('{"k": 5}', "k")[0].ok() and not C.get_base64_config('{}', "k")[0].ok()


@settings(max_examples=60, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])
@given(steps=st.lists(st.tuples(st.sampled_from(["insert", "erase", "clear"]), st.integers(0, 400), st.integers(1, 120)), min_size=1, max_size=30),
       grow=st.sampled_from([0.0, 0.25, 0.5, 0.8, 3.0]), shrink=st.sampled_from([0.0, 0.1, 0.3]), expected=st.sampled_from([0, 500]))
def test_index_ratios_never_lose_a_key_and_the_byte_count_follows_the_buckets(steps, grow, shrink, expected):
    """Whatever grow / shrink ratios and whatever sequence of inserts, erases and clears: a scan by cursor sees exactly
    the live keys, the load stays under the configured limit, the layout epoch moves exactly when the bucket count
    does, and the table's byte count moves by 16 bytes per bucket with it."""
    hc = C.HostTableConfig()
    hc.dim, hc.n_shards = DIM, 1
    hc.index_grow_ratio, hc.index_shrink_ratio, hc.expected_max_items = grow, shrink, expected
    t = C.HostTable(hc)
    t.create_shard(0)
    buckets = lambda: t.export_shard(0, 0, 1 << 30, False)[2]
    live = set()
    limit = min(max(grow, 0.25), 0.85) if grow else 0.5
    for what, start, count in steps:
        b0, e0, m0 = buckets(), t.layout_epoch(0), t.memory_usage()
        keys = np.arange(start, start + count, dtype=np.int64) * 3 - 200
        rows_before = t.size()
        if what == "insert":
            assert t.set_rows(keys, np.ones((count, DIM), F), True).ok()
            live |= set(keys.tolist())
        elif what == "erase":
            assert t.erase_keys(keys) == len(live & set(keys.tolist()))
            live -= set(keys.tolist())
        else:
            t.clear()
            t.create_shard(0)
            live.clear()
        b1 = buckets()
        assert t.size() == len(live) and len(live) <= limit * b1 + 1e-9
        assert (t.layout_epoch(0) != e0) == (b1 != b0) or what == "clear" or (what == "insert" and b1 == b0 and t.layout_epoch(0) != e0)
        if what != "clear":
            rows_grew = t.memory_usage() - m0 - 16 * (b1 - b0)
            assert rows_grew >= 0 and rows_grew % (DIM * 4) == 0          # what is not index is row pool, which only grows
            if what == "erase":
                assert rows_grew == 0
        seen, cursor, finished = [], 0, False
        while not finished:
            k, _, cursor, finished = t.export_shard(0, cursor, 37, False)
            seen += k.tolist()
        assert sorted(seen) == sorted(live)


_cfg_values = st.one_of(st.none(), st.booleans(), st.integers(-(2 ** 40), 2 ** 40), st.floats(allow_nan=False, allow_infinity=False, width=32),
                        st.text(max_size=12), st.lists(st.integers(-5, 5), max_size=3),
                        st.dictionaries(st.sampled_from(["expected_max_items", "grow_ratio", "shrink_ratio", "storage_id", "x"]),
                                        st.one_of(st.integers(-10, 10 ** 7), st.floats(-5, 5), st.text(max_size=4)), max_size=3))
_cfg_keys = ["dim", "optimizer", "lr", "eps", "init_range", "init_accumulator", "sync", "seed", "partition", "backend", "memory_limit",
             "expected_max_items", "grow_ratio", "shrink_ratio", "pool_hash_map", "google_dense_hash_map", "pmem_create_storage",
             "retain_local_image", "alpha", "beta", "l1", "l2", "beta1", "beta2", "weight_decay", "capacity", "max_rows"]


@pytest.fixture(scope="module")
def one_server():
    from parameter_server_b200 import service as S
    master = S.Master()
    server = S.Server(master.address())
    client = S.Client(master.address())
    yield S, server, client
    server.stop()
    master.stop()


@settings(max_examples=120, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(cfg=st.dictionaries(st.sampled_from(_cfg_keys), _cfg_values, max_size=8))
def test_no_storage_config_takes_a_server_down(one_server, cfg):
    """Whatever a client writes into a storage config - wrong types, absurd numbers, nested junk under the
    reference's section names - the answer is a status: the table works, or it is refused; the server lives."""
    import json
    S, server, client = one_server
    cfg = dict(cfg)
    if cfg.get("backend") == "gpu":
        cfg.pop("backend")                                   # no device here: that refusal is tested elsewhere
    st_, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({server.node_id(): [0, 1]}, cfg))
    if st_.ok():
        _, hq = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
        _, hp = client.register_handler("pull", S.LIB, "SparseTablePullOperator", "{}", sid)
        push, pull = S.PushHandler(client, sid, hq), S.PullHandler(client, sid, hp)
        dim = pull.dim()
        assert 1 <= dim <= 65536
        if dim <= 256:
            keys = np.array([1, 2, 3, 2], dtype=np.int64)
            s1 = push.async_push(keys, np.ones((4, dim), F), 5000)
            s2, rows = pull.pull(keys, 5000, False)
            assert rows.shape == (4, dim)                    # a status either way (a memory_limit of 1 byte parks the push and refuses the pull)
        assert client.delete_storage(sid).ok()
    assert not server.exited()


_op_classes = ["SparseTablePullOperator", "SparseTablePushOperator", "ForEachOperator", "ForEachWriteOperator", "EraseIfOperator",
               "DumpOperator", "LoadOperator", "KVSyncOperator", "ShardUpdateContextOperator", "UDFOperator", "RestoreOperator"]
_op_cfg = st.dictionaries(st.sampled_from(["read_only", "max_request_merge_num", "node_selection", "compress_algorithm", "block_size",
                                           "block_serialized_size", "sync_table", "function", "optimizer", "lr", "section"]),
                          st.one_of(st.none(), st.booleans(), st.integers(-(2 ** 33), 2 ** 33), st.text(max_size=8),
                                    st.lists(st.dictionaries(st.sampled_from(["model_name", "table_name", "op_key", "x"]), st.text(max_size=6), max_size=3), max_size=2)),
                          max_size=5)
_carried = st.dictionaries(st.sampled_from(["type", "mod", "rem", "threshold", "section", "factor", "limit", "value", "junk"]),
                           st.one_of(st.none(), st.booleans(), st.integers(-(2 ** 40), 2 ** 40), st.floats(allow_nan=False, allow_infinity=False),
                                     st.sampled_from(["key_mod", "l2_below", "slot0_below", "all", "scale", "clip", "fill", "nonsense"]),
                                     st.lists(st.integers(0, 3), max_size=2)), max_size=6)


@settings(max_examples=100, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(op=st.sampled_from(_op_classes), cfg=_op_cfg, carried=_carried)
def test_no_operator_config_or_carried_item_takes_a_server_down(one_server, op, cfg, carried):
    """Handlers registered with junk configs are refused or work; scans with junk carried items answer with a status;
    the table keeps its rows unless a well-formed scan changed them, and the server lives."""
    import json
    S, server, client = one_server
    st_, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                     S.storage_config({server.node_id(): [0, 1, 2]}, dict(dim=4, optimizer="adagrad", lr=0.1, init_range=0.0)))
    assert st_.ok()
    try:
        _, hq = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
        keys = np.arange(50, dtype=np.int64)
        assert S.PushHandler(client, sid, hq).async_push(keys, np.ones((50, 4), F), 5000).ok()
        st_, hid = client.register_handler("probe", S.LIB, op, json.dumps(cfg), sid)
        if st_.ok():
            text = json.dumps(carried)
            if op in ("ForEachOperator", "ForEachWriteOperator"):
                S.ForEachHandler(client, sid, hid).for_each_raw(text)
            elif op == "EraseIfOperator":
                S.EraseIfHandler(client, sid, hid).erase_if(text)
            elif op == "SparseTablePullOperator":
                st2, rows = S.PullHandler(client, sid, hid).pull(keys, 5000, False)
                assert rows.shape == (50, 4)
            elif op == "SparseTablePushOperator":
                S.PushHandler(client, sid, hid).async_push(keys, np.ones((50, 4), F), 5000)
        info = client.query_storage_info(sid)
        assert info[0].ok() and sum(i.item_number for i in info[1]) <= 50
    finally:
        assert client.delete_storage(sid).ok()
    assert not server.exited()


@pytest.fixture(scope="module")
def dumps_to_damage(one_server, tmp_path_factory):
    """One small table dumped in every format / compression: the raw material of the next test."""
    import json
    S, server, client = one_server
    st_, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                     S.storage_config({server.node_id(): [0, 1]}, dict(dim=4, optimizer="adagrad", lr=0.1, init_range=0.01)))
    assert st_.ok()
    _, hq = client.register_handler("push", S.LIB, "SparseTablePushOperator", "{}", sid)
    keys = np.arange(1, 400, dtype=np.int64) * 1_000_003
    assert S.PushHandler(client, sid, hq).async_push(keys, np.ones((len(keys), 4), F), 5000).ok()
    out = {}
    for fmt in ("binary", "archiveline"):
        for algo in ("", "zstd", "lz4"):
            _, hd = client.register_handler(f"dump_{fmt}_{algo}", S.LIB, "DumpOperator", json.dumps({"compress_algorithm": algo}), sid)
            d = tmp_path_factory.mktemp(f"dump_{fmt}_{algo or 'plain'}")
            st_, n = S.DumpHandler(client, sid, hd).dump(str(d) + "?format=" + fmt, 1)
            assert st_.ok() and n == len(keys)
            out[(fmt, algo)] = (d, {p.name: p.read_bytes() for p in d.iterdir()})
    return out


@settings(max_examples=120, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(fmt=st.sampled_from(["binary", "archiveline"]), algo=st.sampled_from(["", "zstd", "lz4"]),
       flips=st.lists(st.tuples(st.integers(0, 1 << 20), st.integers(0, 255)), max_size=6), cut=st.integers(0, 1 << 20),
       junk=st.binary(max_size=64))
def test_damaged_dump_files_are_refused_or_loaded_never_followed_off_a_cliff(one_server, dumps_to_damage, fmt, algo, flips, cut, junk):
    """Bytes of a dump are flipped, its tail is cut or replaced by junk: the load answers with a status (a flipped
    value may well load) and the server goes on serving."""
    import json
    S, server, client = one_server
    d, files = dumps_to_damage[(fmt, algo)]
    for name, data in files.items():
        b = bytearray(data)
        for pos, val in flips:
            if b:
                b[pos % len(b)] = val
        b = b[:cut % (len(b) + 1)] + junk
        (d / name).write_bytes(bytes(b))
    st_, sid = client.create_storage(S.LIB, "SparseTableStorageOperator",
                                     S.storage_config({server.node_id(): [0, 1, 2]}, dict(dim=4, optimizer="adagrad", lr=0.1, init_range=0.01)))
    assert st_.ok()
    try:
        _, hl = client.register_handler("load", S.LIB, "LoadOperator", json.dumps({"compress_algorithm": algo, "block_size": 64}), sid)
        st_, n = S.LoadHandler(client, sid, hl).load(str(d) + "?format=" + fmt, 2, 20000)
        assert st_.ok() or st_.code() != 0
        info = client.query_storage_info(sid)
        assert info[0].ok() and sum(i.item_number for i in info[1]) <= 10 * 400
    finally:
        assert client.delete_storage(sid).ok()
        for name, data in files.items():
            (d / name).write_bytes(data)
    assert not server.exited()
