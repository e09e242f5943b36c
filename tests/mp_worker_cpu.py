"""Worker of the CPU multi-process tests (gloo): the collective sparse / dense API on the host back-end against a
single-process oracle that sees the concatenation of every rank's batch (same checks as the GPU worker)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from parameter_server_b200 import SparseTable  # noqa: E402
from parameter_server_b200.ops.dense import DenseTable  # noqa: E402


def gather(obj):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj)
    return out


def elastic(rank, world):
    """Reshard, 2x replication (sync / restore) and dump / load of a host table, 3 ranks."""
    import tempfile
    from parameter_server_b200.parallel import ReplicaSet, checkpoint, reshard

    dim, n_shards = 4, 7
    kw = dict(lr=0.1, init_accumulator=0.2)
    t = SparseTable(dim, "adagrad", kw, n_shards=n_shards, device="cpu")
    rng = np.random.default_rng(11)                   # the same keys on every rank: everybody can check everything
    keys = torch.from_numpy(rng.choice(1 << 30, size=900, replace=False).astype(np.int64))
    mine = keys[rank::world]
    t.pull(mine)
    t.push(torch.from_numpy(np.random.default_rng(rank).standard_normal((mine.numel(), dim)).astype(np.float32)))
    want = t.pull(keys, insert=False)
    total = sum(gather(t.size()))
    assert total == 900, total
    # rebalance: everything to rank 0 and 1, then a rotation; reads in the middle of the move still see every row
    seen = []
    for new_owner in ([s % 2 for s in range(n_shards)], [(s + 1) % world for s in range(n_shards)]):
        reshard(t, new_owner, between_rounds=lambda: seen.append(torch.equal(t.pull(keys, insert=False), want)))
        assert list(t.shard_owner) == new_owner
        assert torch.equal(t.pull(keys, insert=False), want)
        sizes = gather(t.size()); assert sum(sizes) == 900, (sizes, new_owner, t.table.shard_list())
        for k, _ in t.export():
            owners = {new_owner[int(s)] for s in __import__("parameter_server_b200").C.sparse_shards_of(k.numpy(), n_shards)}
            assert owners <= {rank}, owners
    assert seen == [True, True], seen
    # 2x replication: full sync, an incremental one after a small push, then rank 1 loses its table
    rep = ReplicaSet(t)
    sent = gather(rep.sync())
    assert sum(sent) == 900, sent
    some = keys[:40]
    t.pull(some)
    t.push(torch.ones(40, dim))
    want = t.pull(keys, insert=False)
    sent = gather(rep.sync())
    assert sum(sent) == 40, sent
    assert sum(gather(rep.sync())) == 0
    lost = 1
    before = t.size()
    if rank == lost:
        t.table.clear()
        assert t.size() == 0
    got = rep.restore(lost)
    if rank == lost:
        assert got == before and t.size() == before
    assert torch.equal(t.pull(keys, insert=False), want)
    # dump with 2 files per rank, load into a table with another shard count; one rank's files alone restore that rank
    uri = [tempfile.mkdtemp(prefix="psb_ckpt_") if rank == 0 else None]
    dist.broadcast_object_list(uri, src=0)
    written = gather(checkpoint.dump(t, uri[0], file_number=2))
    assert sum(written) == 900, written
    t2 = SparseTable(dim, "adagrad", kw, n_shards=5, device="cpu")
    landed = gather(checkpoint.load(t2, uri[0], batch=128))
    assert sum(landed) == 900 and sum(gather(t2.size())) == 900, landed
    assert torch.equal(t2.pull(keys, insert=False), want)
    if rank == lost:
        t.table.clear()
    dist.barrier()
    checkpoint.load(t, uri[0], only_node=lost)
    assert torch.equal(t.pull(keys, insert=False), want)
    dist.barrier()
    if rank == 0:
        import shutil
        shutil.rmtree(uri[0], ignore_errors=True)


def scans(rank, world):
    """for_each / for_each_write / erase_if of the collective table: every rank scans its own entries, the answers
    are combined over the ranks."""
    dim = 4
    t = SparseTable(dim, "adagrad", dict(lr=0.1, init_accumulator=0.5), n_shards=5, device="cpu", init_range=0.0)
    keys = torch.arange(1, 1201, dtype=torch.int64)
    mine = keys[rank::world]
    t.pull(mine)
    t.push(-(mine % 7 + 1).float()[:, None] * torch.ones(1, dim))            # row = +lr * g / sqrt(acc): depends on key % 7
    want = t.pull(keys, insert=False)
    st = t.for_each(collective=True)
    assert st["count"] == 1200 and abs(st["sum"] - float(want.double().sum())) < 1e-6 * abs(st["sum"])
    assert abs(st["max_abs"] - float(want.abs().max())) < 1e-12
    acc = t.for_each(section=1, collective=True)
    assert acc["count"] == 1200 and acc["sum"] > 0.5 * 1200 * dim
    info = t.storage_info(collective=True)
    assert sorted(r["shard_id"] for r in info) == list(range(5)) and sum(r["item_number"] for r in info) == 1200
    assert all(r["node_id"] == t.shard_owner[r["shard_id"]] for r in info) and len(t.storage_info()) == len([s for s in range(5) if t.shard_owner[s] == rank])
    # a user reducer: the largest key that this rank holds; merged by the caller
    parts = t.for_each(lambda k, r: int(k.max()))
    assert max(max(p) if p else 0 for p in gather(parts)) == 1200
    # writing scan: halve the embeddings of even keys, everywhere
    def halve(k, r):
        new = r.clone()
        new[k % 2 == 0, :dim] *= 0.5
        return new
    assert t.for_each_write(halve, collective=True) == 600
    got = t.pull(keys, insert=False)
    even = keys % 2 == 0
    assert torch.equal(got[even], 0.5 * want[even]) and torch.equal(got[~even], want[~even])
    assert t.for_each(section=1, collective=True)["sum"] == acc["sum"]        # the slots were left alone
    assert t.for_each_write(lambda k, r: None) == 0
    # erase_if: a built-in predicate, then a torch predicate over keys and rows
    assert t.erase_if({"type": "key_mod", "mod": 3, "rem": 0}, collective=True) == 400
    small = float(got.norm(dim=1).median())
    n = t.erase_if(lambda k, r: r[:, :dim].norm(dim=1) < small, collective=True)
    left = keys[keys % 3 != 0]
    assert n == int((got[keys % 3 != 0].norm(dim=1) < small).sum()) and sum(gather(t.size())) == len(left) - n
    assert t.erase_if({"type": "all"}, collective=True) == len(left) - n and sum(gather(t.size())) == 0
    try:
        t.erase_if({"type": "nonsense"})
        raise AssertionError("an unknown predicate must be refused")
    except ValueError:
        pass
    dist.barrier()


def predictor_sync(rank, world):
    """Every rank ships the rows of its own shards to one predictor table of the service layer."""
    import json
    from parameter_server_b200 import service as S
    from parameter_server_b200.parallel import PredictorSync

    dim = 4
    cluster = None
    info = [None]
    if rank == 0:                                     # the serving side lives in rank 0's process, reachable over TCP
        master = S.Master()
        servers = [S.Server(master.address()) for _ in range(2)]
        admin = S.Client(master.address())
        ids = [s.node_id() for s in servers]
        cfg = dict(dim=dim, optimizer="set", init_range=0.0)
        st, sid = admin.create_storage(S.LIB, "SparseTableStorageOperator", S.storage_config({ids[0]: [0, 1], ids[1]: [2]}, cfg))
        assert st.ok(), st
        _, h_pull = admin.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", json.dumps({"read_only": True}), sid)
        _, h_sync = admin.register_handler("sync", S.LIB, "KVSyncOperator", json.dumps({"block_size": 50}), sid)
        cluster = (master, servers, admin)
        info = [(master.address(), sid, h_pull, h_sync)]
    dist.broadcast_object_list(info, src=0)
    addr, sid, h_pull, h_sync = info[0]
    client = S.Client(addr)
    assert client.initialize_storage(sid).ok()
    t = SparseTable(dim, "sgd", dict(lr=1.0), n_shards=2 * world + 1, device="cpu", init_range=0.0)
    keys = torch.arange(1, 901, dtype=torch.int64)
    mine = keys[rank::world]
    t.pull(mine)
    t.push(-(mine % 9 + 1).float()[:, None] * torch.ones(1, dim))
    sync = PredictorSync(t, S.SyncHandler(client, sid, h_sync), embedding_only=True)
    sent = gather(sync.sync())
    assert sum(sent) == 900 and all(n > 0 for n in sent), sent              # every rank sent its own rows only
    want = t.pull(keys, insert=False)
    dist.barrier()
    st, rows = S.PullHandler(client, sid, h_pull).pull(keys.numpy())
    assert st.ok() and np.array_equal(rows, want.numpy())
    some = keys[:30]
    t.pull(some[rank::world])
    t.push(torch.ones(some[rank::world].numel(), dim))
    assert sum(gather(sync.sync())) == 30
    want = t.pull(keys, insert=False)
    dist.barrier()
    st, rows = S.PullHandler(client, sid, h_pull).pull(keys.numpy())
    assert st.ok() and np.array_equal(rows, want.numpy())
    dist.barrier()
    if cluster is not None:
        for s_ in cluster[1]:
            s_.stop()
        cluster[0].stop()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    for dim, opt, kw, bag in [(8, "adagrad", dict(lr=0.05, init_accumulator=0.1), 1), (4, "sgd", dict(lr=0.5), 2),
                              (8, "adam", dict(lr=0.01), 1)]:
        n_shards = 2 * world + 1
        t = SparseTable(dim, opt, kw, n_shards=n_shards, device="cpu")
        ref = SparseTable(dim, opt, kw, n_shards=n_shards, device="cpu", group="none") if rank == 0 else None
        rng = np.random.default_rng(5 + rank)
        for step in range(4):
            keys = torch.from_numpy((rng.zipf(1.2, size=600).astype(np.int64) * 7919) % 3000)
            grads = torch.from_numpy(rng.standard_normal((600 // bag, dim)).astype(np.float32) * 1e-2)
            out = t.pull(keys, bag_size=bag, mean=(bag > 1))
            t.push(grads, bag_size=bag, mean=(bag > 1))
            all_keys, all_grads, all_out = gather(keys), gather(grads), gather(out)
            if rank == 0:
                want = ref.pull(torch.cat(all_keys), bag_size=bag, mean=(bag > 1))
                got = torch.cat(all_out)
                assert torch.allclose(got, want, rtol=1e-5, atol=1e-7), (opt, step, (got - want).abs().max())
                ref.push(torch.cat(all_grads), bag_size=bag, mean=(bag > 1))
        sizes = gather(t.size())
        if rank == 0:
            assert sum(sizes) == ref.size(), (sizes, ref.size())
        # every rank holds only keys of its own shards
        for k, _ in t.export():
            owners = {t.shard_owner[__import__("parameter_server_b200").C.sparse_shard_of(int(x), n_shards)] for x in k.tolist()}
            assert owners <= {rank}, owners
    elastic(rank, world)
    scans(rank, world)
    predictor_sync(rank, world)
    # dense table: all-reduce + optimizer on every rank, identical parameters everywhere
    d = DenseTable({"w": (64, 8), "b": (64,)}, "adamw", dict(lr=1e-2, weight_decay=0.01), device="cpu")
    d.load({"w": torch.ones(64, 8), "b": torch.zeros(64)})
    for step in range(3):
        d.zero_grads()
        d.grads["w"].add_(torch.full((64, 8), float(rank + 1 + step)))
        d.grads["b"].add_(torch.full((64,), 0.5 * (rank + 1)))
        d.push()
    sigs = gather((float(d.pull("w").sum()), float(d.pull("b").sum())))
    assert all(s == sigs[0] for s in sigs), sigs
    # checkpoint of the dense table: every rank writes its slice; a table of the same job and a single-process
    # table (another world size) resume from it and take the next step exactly like the original
    import tempfile
    from parameter_server_b200.parallel import checkpoint
    ck = [tempfile.mkdtemp(prefix="psb_dense_") if rank == 0 else None]
    dist.broadcast_object_list(ck, src=0)
    wrote = gather(checkpoint.dump_dense(d, ck[0]))
    assert sum(wrote) == d.numel, wrote
    d2 = DenseTable({"w": (64, 8), "b": (64,)}, "adamw", dict(lr=1e-2, weight_decay=0.01), device="cpu")
    assert checkpoint.load_dense(d2, ck[0]) == d.numel and d2.step_count == d.step_count
    solo = DenseTable({"w": (64, 8), "b": (64,)}, "adamw", dict(lr=1e-2, weight_decay=0.01), device="cpu", group="none")
    checkpoint.load_dense(solo, ck[0])
    for t_ in (d, d2):
        t_.zero_grads()
        t_.grads["w"].add_(torch.full((64, 8), 0.25))
        t_.push()
    solo.zero_grads()
    solo.grads["w"].add_(torch.full((64, 8), 0.25 * world))               # what the three ranks sum to
    solo.push(grad_scale=1.0 / world)
    assert torch.equal(d.pull("w"), d2.pull("w")) and torch.equal(d.pull("b"), d2.pull("b"))
    assert torch.allclose(d.pull("w"), solo.pull("w"), rtol=0, atol=1e-7)
    dist.barrier()
    if rank == 0:
        import shutil
        shutil.rmtree(ck[0], ignore_errors=True)
    assert d.pull("w").mean().item() < 1.0           # the weights moved against the (positive) gradient
    dist.barrier()
    if rank == 0:
        print("cpu collective ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
