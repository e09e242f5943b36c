"""Worker of the multi-GPU tests: started once per GPU by torch.distributed.run.

Checks the fused sparse pull / push and the fused dense push at world > 1 against a CPU oracle that
sees the concatenation of every rank's batch, then runs DLRM steps. NVLS is irrelevant here (the
kernels use plain peer loads / stores)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from parameter_server_b200 import SparseTable  # noqa: E402
from blocked_sum import blocked_segment_sum  # noqa: E402
from parameter_server_b200.ops.dense import DenseTable  # noqa: E402


def mostly_close(got, ref, rtol, atol, loose_atol, frac=0.999):
    """Every element within the loose bound and at least ``frac`` of them within the tight one. With more than
    two ranks the cross-rank gradient fold uses atomics, so sums differ from the oracle in the last bits; Adam
    divides by sqrt(v) + eps and turns that into a visible difference where a summed gradient is almost zero."""
    d = (got - ref).abs()
    tight = d <= atol + rtol * ref.abs()
    return bool(tight.float().mean() >= frac) and bool((d <= loose_atol + rtol * ref.abs()).all())


def gather(obj):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj)
    return out


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    which = sys.argv[1] if len(sys.argv) > 1 else "all"

    if which in ("all", "sparse"):
        # Twice: with the default (atomic) duplicate sums, compared within a tolerance, and in reproducible mode, where
        # every rank sums its duplicates in position order and the owners fold the ranks in rank order: then the tables
        # must equal, bit for bit, an oracle that adds in that same order.
        # A third time with the gradient rows crossing NVLink as bf16: every rank's partial sum is rounded once (relative
        # error 2^-9 of a sum that reaches 0.5 for the head keys), so the comparison is looser, in proportion to the
        # number of ranks that contribute.
        for mode in ("atomic", "ordered", "bf16wire"):
            deterministic = mode == "ordered"
            wire16 = mode == "bf16wire"
            for dim, opt, kw in [(64, "adagrad", dict(lr=0.05, init_accumulator=0.1)), (16, "sgd", dict(lr=0.5)),
                                 (128, "adam", dict(lr=0.01))]:
                if wire16 and opt == "adam":
                    continue   # Adam divides by sqrt(v): a rounded gradient near zero moves the update visibly
                n_shards = world * 3 + 1
                g = SparseTable(dim, opt, kw, n_shards=n_shards, capacity=1 << 16, max_keys=1 << 15, wait_limit_s=5.0)
                g.set_deterministic(deterministic)
                g.set_grad_wire_bf16(wire16)
                c = SparseTable(dim, opt, kw, n_shards=n_shards, device="cpu", group="none") if rank == 0 else None
                if c is not None:
                    c.world, c.rank = 1, 0
                    for s in range(n_shards):
                        c.table.create_shard(s)
                rng = np.random.default_rng(100 + rank)
                for step in range(4):
                    n = 20000
                    keys = torch.from_numpy((rng.zipf(1.1, size=n).astype(np.int64) * 7919) % 50000)
                    grads = torch.from_numpy(rng.standard_normal((n, dim)).astype(np.float32) * 1e-2)
                    out = g.pull(keys.cuda())
                    g.push(grads.cuda())
                    g.check()
                    all_keys, all_grads, all_out = gather(keys), gather(grads), gather(out.cpu())
                    if rank == 0:
                        ck = torch.cat(all_keys)
                        ref = c.pull(ck)
                        got = torch.cat(all_out)
                        if deterministic:
                            assert torch.equal(got, ref), f"pull differs dim={dim} step={step}: {(got-ref).abs().max()}"
                            # the oracle adds like the kernels: per rank in the blocked position order, then the ranks in rank order
                            us, aggs = [], []
                            for k_r, g_r in zip(all_keys, all_grads):
                                u, agg = blocked_segment_sum(k_r.numpy(), g_r.numpy())
                                us.append(torch.from_numpy(u)); aggs.append(torch.from_numpy(agg))
                            c.push(torch.cat(aggs), keys=torch.cat(us))
                        elif wire16:
                            assert mostly_close(got, ref, 2e-2, 1e-3 * world, 5e-3 * world), \
                                f"pull mismatch (bf16 wire) dim={dim} step={step}: {(got-ref).abs().max()}"
                            c.push(torch.cat(all_grads))
                        else:
                            assert mostly_close(got, ref, 1e-3, 2e-5, 2e-3 if opt == "adam" else 2e-5), \
                                f"pull mismatch dim={dim} step={step}: {(got-ref).abs().max()}"
                            c.push(torch.cat(all_grads))
                # final table state: every rank exports its local rows; rank 0 compares with the oracle
                ks, rs = [], []
                for k, r in g.export():
                    ks.append(k.cpu()); rs.append(r.cpu())
                ks = torch.cat(ks) if ks else torch.empty(0, dtype=torch.int64)
                rs = torch.cat(rs) if rs else torch.empty(0, g.table.stride())
                owners = set(int(g.shard_owner[int(x)]) for x in
                             [__import__("parameter_server_b200").C.sparse_shard_of(int(k), n_shards) for k in ks[:200].tolist()])
                assert owners <= {rank}, f"rank {rank} holds foreign keys: {owners}"
                all_ks, all_rs = gather(ks), gather(rs)
                if rank == 0:
                    K, R = torch.cat(all_ks), torch.cat(all_rs)
                    assert K.numel() == torch.unique(K).numel() == c.size(), (K.numel(), c.size())
                    ref, found = c.get_rows(K, emb_only=False)
                    assert found.all()
                    if deterministic:
                        assert torch.equal(R, ref), f"table differs from the oracle, {opt}: {(R-ref).abs().max()}"
                    elif wire16:
                        assert mostly_close(R, ref, 2e-2, 1e-3 * world, 1e-2 * world), f"table mismatch (bf16 wire) {opt}: {(R-ref).abs().max()}"
                    else:
                        assert mostly_close(R, ref, 2e-3, 1e-4, 4e-3 if opt == "adam" else 1e-4), f"table mismatch {opt}: {(R-ref).abs().max()}"
                dist.barrier()
        if rank == 0:
            print("sparse ok", flush=True)

    if which in ("all", "dense"):
        for gdt in (torch.float32, torch.bfloat16):
            shapes = {"a": (300, 40), "b": (77,), "c": (1024, 64)}
            t = DenseTable(shapes, "adamw", dict(lr=1e-2, weight_decay=0.01), grad_dtype=gdt, wait_limit_s=5.0)
            gen = torch.Generator().manual_seed(0)
            init = {k: torch.randn(v, generator=gen) for k, v in shapes.items()}
            t.load(init)
            ref = {k: v.clone() for k, v in init.items()}
            m = {k: torch.zeros_like(v) for k, v in init.items()}
            vv = {k: torch.zeros_like(v) for k, v in init.items()}
            for step in range(1, 4):
                local = {k: torch.randn(v, generator=torch.Generator().manual_seed(10 * step + rank)) for k, v in shapes.items()}
                for k in shapes:
                    t.grads[k].copy_(local[k].to(gdt))
                t.push()
                t.check()
                alls = gather({k: v.to(gdt).float() for k, v in local.items()})
                for k in shapes:
                    gsum = sum(a[k] for a in alls) / world
                    m[k] = 0.9 * m[k] + 0.1 * gsum
                    vv[k] = 0.999 * vv[k] + 0.001 * gsum * gsum
                    ref[k] = ref[k] * (1 - 1e-2 * 0.01)
                    ref[k] = ref[k] - 1e-2 * (m[k] / (1 - 0.9 ** step)) / ((vv[k] / (1 - 0.999 ** step)).sqrt() + 1e-8)
                for k in shapes:
                    got = t.pull(k).float().cpu()
                    assert torch.allclose(got, ref[k].bfloat16().float(), rtol=2e-2, atol=2e-2), (k, step, (got - ref[k]).abs().max())
            dist.barrier()
        if rank == 0:
            print("dense ok", flush=True)

    if which in ("all", "migrate"):
        from parameter_server_b200.parallel import ReplicaSet, reshard
        n_shards = 2 * world
        t = SparseTable(32, "adagrad", dict(lr=0.05, init_accumulator=0.1), n_shards=n_shards, capacity=1 << 16,
                        max_keys=1 << 15, wait_limit_s=5.0)
        rng = np.random.default_rng(7 + rank)
        keys = torch.from_numpy(rng.integers(0, 1 << 40, size=20000)).cuda()
        t.pull(keys)
        t.push(torch.randn(20000, 32, device="cuda") * 1e-2)
        before = t.pull(keys).clone()
        t.check()
        total_before = sum(gather(t.size()))
        # rebalance: rotate the ownership of every shard by one rank
        new_owner = [(o + 1) % world for o in t.shard_owner]
        reads = []

        def read_during():      # reads stay served while rows are on the move
            reads.append(bool(torch.equal(t.pull(keys, insert=False, for_push=False), before)))

        reshard(t, new_owner, batch=4096, between_rounds=read_during)
        t.check()
        assert reads and all(reads), reads
        assert sum(gather(t.size())) == total_before
        ks = torch.cat([k for k, _ in t.export()] or [torch.empty(0, dtype=torch.int64, device="cuda")])
        owners = {new_owner[__import__("parameter_server_b200").C.sparse_shard_of(int(k), n_shards)] for k in ks[:500].tolist()}
        assert owners <= {rank}, owners
        after = t.pull(keys, insert=False)
        t.check()
        assert torch.equal(after, before), "rows changed while moving between GPUs"
        # 2x replication: mirror on the partner, incremental sync, restore after a loss
        rs = ReplicaSet(t)
        n0 = t.size()
        assert rs.sync() == n0 and rs.mirror.size() == gather(n0)[(rank - 1) % world]
        t.pull(keys[:100]); t.push(torch.ones(100, 32, device="cuda") * 1e-2); t.check()
        assert 0 < rs.sync() <= 100 * world          # only what changed travels (keys of this rank's shards)
        want = t.pull(keys, insert=False).clone()
        if rank == 0:
            t.clear()                                  # rank 0 "lost" its HBM contents
        got = rs.restore(0)
        if rank == 0:
            assert got == n0 and t.size() == n0
        again = t.pull(keys, insert=False)
        t.check()
        assert torch.equal(again, want)
        # replication inside the push: the mirror on the partner is exact after every push, so a table that is lost
        # BETWEEN two steps, with no sync() ever called, comes back bit for bit
        t3 = SparseTable(32, "adagrad", dict(lr=0.05, init_accumulator=0.1), n_shards=n_shards, capacity=1 << 16,
                         max_keys=1 << 15, wait_limit_s=5.0, replicate=True)
        rs3 = ReplicaSet(t3, in_push=True)
        zk = torch.from_numpy((rng.zipf(1.1, size=20000).astype(np.int64) * 7919) % 30000).cuda()
        for _ in range(3):
            t3.pull(zk); t3.push(torch.randn(20000, 32, device="cuda") * 1e-2)
        t3.check()
        mine = torch.cat([k for k, _ in t3.export()] or [torch.empty(0, dtype=torch.int64, device="cuda")])
        want3, _ = t3.get_rows(mine, emb_only=False)
        n3 = t3.size()
        assert rs3.mirror.size() == gather(n3)[(rank - 1) % world]
        if rank == 0:
            t3.clear()
        got3 = rs3.restore(0)
        if rank == 0:
            assert got3 == n3 == t3.size()
        back3, found3 = t3.get_rows(mine, emb_only=False)
        t3.check()
        assert found3.all() and torch.equal(back3, want3), "the replica kept by the push is not exact"
        t3.pull(zk); t3.push(torch.randn(20000, 32, device="cuda") * 1e-2); t3.check()     # and training goes on
        dist.barrier()
        # dump with 2 files per rank, load into a table with another shard count (rehash) and from all ranks' files
        from parameter_server_b200.parallel import checkpoint
        import tempfile
        box = [tempfile.mkdtemp(prefix="psb_dump_") if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        assert checkpoint.dump(t, box[0], file_number=2) == t.size()
        t2 = SparseTable(32, "adagrad", dict(lr=0.05, init_accumulator=0.1), n_shards=3 * world, capacity=1 << 16,
                         max_keys=1 << 15, wait_limit_s=5.0)
        checkpoint.load(t2, box[0])
        assert sum(gather(t2.size())) == total_before
        assert torch.equal(t2.pull(keys, insert=False), want)
        t2.check()
        dist.barrier()
        if rank == 0:
            import shutil
            shutil.rmtree(box[0], ignore_errors=True)
            print("migrate ok", flush=True)

    if which in ("all", "aggemm"):
        from parameter_server_b200.ops import gemm as G
        N, K, M = 512 * world, 384, 1000
        t = DenseTable({"w": (N, K)}, "sgd", dict(lr=0.5), grad_dtype=torch.float32, wait_limit_s=5.0, scatter_peers=False)
        gen = torch.Generator().manual_seed(3)
        w0 = torch.randn(N, K, generator=gen) * 0.1
        t.load({"w": w0})
        ref_w = w0.clone()
        for step in range(3):
            local_g = torch.randn(N, K, generator=torch.Generator().manual_seed(50 * step + rank))
            t.grads["w"].copy_(local_g)
            t.push()
            gsum = sum(gather(local_g)) / world
            ref_w = ref_w - 0.5 * gsum
            x = (torch.randn(M, K, generator=torch.Generator().manual_seed(7 + step)) * 0.5).cuda().bfloat16()
            y = G.ag_linear(x, t, "w", gather_ctas=4)
            G.check_gemm_errors()
            ref = x.float().cpu() @ ref_w.bfloat16().float().t()
            err = (y.float().cpu() - ref).abs().max().item()
            assert err < 0.15, f"ag_linear mismatch at step {step}: {err}"
            # the local copy now holds every rank's rows
            assert torch.allclose(t.params["w"].float().cpu(), ref_w.bfloat16().float(), atol=2e-2)
            dist.barrier()
        if rank == 0:
            print("aggemm ok", flush=True)

    if which in ("all", "dlrm"):
        from parameter_server_b200.models import DLRM, DLRMConfig, SyntheticCTR
        cfg = DLRMConfig(vocab_max=5e4)
        model = DLRM(cfg, 1024, table_capacity=1 << 18)
        data = SyntheticCTR(cfg, 1024, pool=4, seed=rank)
        losses = []
        for _ in range(20):
            model.train_step(*data.next())
            losses.append(model.read_loss())
        model.check()
        assert all(np.isfinite(losses)), losses
        # dense parameters stay identical on every rank
        sig = float(model.dense.flat_params.float().sum().item())
        sigs = gather(sig)
        assert max(sigs) - min(sigs) == 0.0, sigs
        # the arrangement used from three ranks on: one stream, but the sparse push beside the dense push
        model2 = DLRM(cfg, 1024, table_capacity=1 << 18, overlap=False, tail_overlap=True)
        assert model2.tail_overlap
        data2 = SyntheticCTR(cfg, 1024, pool=4, seed=rank)
        for i in range(12):
            if i == 4:
                model2.enable_graph()
            model2.train_step(*data2.next())
            l2 = model2.read_loss()
            assert np.isfinite(l2), l2
        model2.check()
        sigs = gather(float(model2.dense.flat_params.float().sum().item()))
        assert max(sigs) - min(sigs) == 0.0, sigs
        if rank == 0:
            print("dlrm ok", [round(x, 3) for x in losses[:3]], "...", round(losses[-1], 3), flush=True)

    if which == "elastic":
        # A rank leaves between two steps; the others learn of it on the host (heartbeat store) before their next
        # launch, rebuild the table on the survivors and refill it from the last dump. No kernel ever waits for
        # the rank that left. (Run with NCCL_NVLS_ENABLE=0; the kernels of this repository use plain peer
        # loads / stores.)
        import shutil
        import tempfile
        from parameter_server_b200.parallel import checkpoint
        from parameter_server_b200.parallel.membership import Membership, RankLost
        t = SparseTable(32, "adagrad", dict(lr=0.05, init_accumulator=0.1), n_shards=2 * world, capacity=1 << 16,
                        max_keys=1 << 14, wait_limit_s=5.0)
        rng = np.random.default_rng(21 + rank)
        keys = torch.from_numpy(rng.integers(0, 1 << 40, size=8000)).cuda()
        for _ in range(2):
            t.pull(keys); t.push(torch.randn(8000, 32, device="cuda") * 1e-2)
        t.check()
        box = [tempfile.mkdtemp(prefix="psb_elastic_") if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        checkpoint.dump(t, box[0], file_number=2)
        mine = [(k.cpu(), r.cpu()) for k, r in t.export()]
        everything = gather(mine)                                   # what the dump must bring back, known to rank 0
        m = Membership(dist.distributed_c10d._get_default_store(), rank, world, timeout_s=2.0, prefix="psb/test_elastic")
        leaver = world - 1
        lost = None
        for step in range(1, 5):
            if rank == leaver and step == 3:
                torch.cuda.synchronize()                            # nothing of this rank is in flight
                m.leave()
                print(f"rank {rank} left", flush=True)
                os._exit(0)
            try:
                m.step(step)
            except RankLost as e:
                lost = e
                break
            t.pull(keys); t.push(torch.randn(8000, 32, device="cuda") * 1e-2)
            t.check()
        assert lost is not None and lost.ranks == [leaver] and lost.left == [leaver], lost
        torch.cuda.synchronize()
        if rank == 0:
            # with two ranks the survivor serves alone: a private table, refilled from every file of the dump
            t2 = SparseTable(32, "adagrad", dict(lr=0.05, init_accumulator=0.1), n_shards=4, capacity=1 << 16,
                             max_keys=1 << 14, group="none")
            n = checkpoint.load(t2, box[0])
            ks = torch.cat([k for part in everything for k, _ in part])
            rs = torch.cat([r for part in everything for _, r in part])
            assert n == ks.numel() == t2.size(), (n, ks.numel(), t2.size())
            got, found = t2.get_rows(ks.cuda(), emb_only=False)
            assert found.all() and torch.equal(got.cpu(), rs)
            out = t2.pull(keys)                                     # and it trains on
            t2.push(torch.zeros(8000, 32, device="cuda")); t2.check()
            assert torch.isfinite(out).all()
            shutil.rmtree(box[0], ignore_errors=True)
            print("elastic ok", flush=True)
        os._exit(0)                                                 # the group lost a member: no collective teardown

    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback
        # one line per rank on stdout, so that the launcher's own noise cannot hide the cause
        print(f"WORKER-FAILED rank {os.environ.get('RANK')}: " + traceback.format_exc().replace("\n", " | ")[-1500:], flush=True)
        os._exit(1)
