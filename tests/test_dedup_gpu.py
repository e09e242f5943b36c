"""Stand-alone dedup + partition against torch.unique and the host partitioner."""
import numpy as np
import pytest
import torch

from parameter_server_b200 import C
from parameter_server_b200.ops.dedup import KeyDeduper

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,world,n_shards", [(1, 1, 1), (1000, 1, 1), (50000, 4, 13), (65536, 8, 8)])
def test_dedup_partition(n, world, n_shards):
    rng = np.random.default_rng(n)
    keys = torch.from_numpy((rng.zipf(1.1, size=n).astype(np.int64) * 7919) % 100003).cuda()
    shard_owner = torch.tensor([s % world for s in range(n_shards)], dtype=torch.int32, device="cuda")
    d = KeyDeduper(1 << 16)
    for _ in range(2):   # the scratch table must be left empty by the first call
        uniq, owner, inverse, counts = d(keys, shard_owner, world)
        ref = torch.unique(keys)
        assert uniq.numel() == ref.numel() == int(counts[0])
        assert torch.equal(torch.sort(uniq)[0], ref)
        assert torch.equal(uniq[inverse.long()], keys)
        exp_owner = torch.tensor([int(shard_owner[C.sparse_shard_of(int(k), n_shards)]) for k in uniq.tolist()[:2000]])
        assert torch.equal(owner[:2000].cpu().long(), exp_owner.long())
        assert torch.equal(counts[1:].cpu().long(), torch.bincount(owner.long(), minlength=world).cpu())
