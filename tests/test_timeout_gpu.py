"""The time-out path of every device-side wait, reached the safe way: a flag that nothing sets.

The reference turns a late peer into ``Status::Timeout`` (pico-ps/common/DistributedAsyncReturn.cpp:46-54) and its
HA test loops ``pull(timeout=100ms)`` until a restarted server answers (pico-ps/test/ps_pmem_test.cpp:367-532).
Here a wait is a bounded spin inside a kernel. Each test wires two engines of one process to each other on ONE GPU,
launches the kernel of rank 0 only, and lets its wait for rank 1 run out after 20 ms: the kernel records a status and
returns, the host maps it to TIMEOUT, and the CUDA context keeps working. Nothing faults, traps or spins without a
limit, and no two kernels ever wait for each other on the same GPU.
"""
import pytest
import torch

from parameter_server_b200 import C, SparseTable, StatusCode
from parameter_server_b200.ops import gemm as G
from parameter_server_b200.ops.optim import make_opt_config

pytestmark = pytest.mark.gpu

LIMIT_S = 0.02


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _sparse_pair(dim=16):
    tables, engines = [], []
    for r in range(2):
        tc = C.GpuTableConfig()
        tc.device = torch.cuda.current_device()
        tc.dim = dim
        tc.opt_type = C.OPT_SGD
        tc.index_capacity = 1 << 13
        tc.slab_shift = 12
        t = C.GpuTable(tc)
        ec = C.SparseEngineConfig()
        ec.world, ec.rank = 2, r
        ec.max_keys = 1 << 12
        ec.n_shards = 2
        ec.wait_limit_s = LIMIT_S
        tables.append(t)
        engines.append(C.SparseEngine(t, ec))
    for e in engines:
        e.connect_local(engines)
    return tables, engines


def test_sparse_pull_wait_for_a_silent_rank_runs_out_with_status_timeout():
    tables, (e0, e1) = _sparse_pair()
    keys = torch.arange(1000, device="cuda")
    out = torch.empty(1000, 16, device="cuda")
    flags = C.FUSED_COPY_ROWS | C.FUSED_INSERT | C.FUSED_PREPARE_PUSH
    assert e0.pull(keys.data_ptr(), 1000, 1, out.data_ptr(), flags, _stream()).ok()     # rank 1 never calls
    st = e0.check(_stream())
    assert st.code() == StatusCode.TIMEOUT and "source rank's keys" in st.msg()
    # the context is alive, the engine refuses launches until every rank has re-armed
    assert float(torch.ones(8, device="cuda").sum()) == 8.0
    assert not e0.pull(keys.data_ptr(), 1000, 1, out.data_ptr(), flags, _stream()).ok()
    assert e0.reset(_stream()).ok() and e1.reset(_stream()).ok()
    assert e0.check(_stream()).ok()
    # after the reset the epochs are aligned again: the same lonely call times out at the same site, not earlier
    assert e0.pull(keys.data_ptr(), 1000, 1, out.data_ptr(), flags, _stream()).ok()
    st = e0.check(_stream())
    assert st.code() == StatusCode.TIMEOUT and "source rank's keys" in st.msg()
    assert e0.reset(_stream()).ok() and e1.reset(_stream()).ok()
    # and a single-rank table on the same device is unaffected
    t = SparseTable(16, "sgd", dict(lr=0.1), device="cuda", capacity=1 << 12, max_keys=1 << 10)
    a = t.pull(keys[:512]); t.push(torch.ones(512, 16, device="cuda")); t.check()
    assert torch.allclose(t.pull(keys[:512], insert=False), a - 0.1)


def test_dense_push_wait_for_a_silent_rank_runs_out_with_status_timeout():
    dev = torch.cuda.current_device()
    engines = [C.DenseEngine(dev, 2, r, 1 << 16, False, C.OPT_SGD, LIMIT_S) for r in range(2)]
    for e in engines:
        e.connect_local(engines)
    opt = make_opt_config("sgd", lr=0.1)
    assert engines[0].step(opt, 1.0, _stream()).ok()                                    # rank 1 never calls
    st = engines[0].check(_stream())
    assert st.code() == StatusCode.TIMEOUT and "peer's gradients" in st.msg()
    assert float(torch.ones(8, device="cuda").sum()) == 8.0
    assert engines[0].reset(_stream()).ok() and engines[0].check(_stream()).ok()


def test_gemm_wait_for_a_gathered_tile_runs_out_and_frees_its_tmem():
    """All-gather + GEMM with nobody gathering (zero gather CTAs): the producer's wait for a remote weight tile runs
    out, the CTA records site 5, frees its TMEM and returns; the next plain GEMM is correct."""
    M, N, K = 256, 512, 256
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    ready = torch.zeros(N // 256, dtype=torch.int32, device="cuda")
    g = dict(gather_peers=[w.data_ptr(), w.data_ptr()], gather_rank=0, rows_per_rank=N // 2, gather_ready=ready.data_ptr(),
             gather_epoch=1, gather_ctas=0)
    G.gemm(x, w, gather=g, wait_limit_s=LIMIT_S)
    with pytest.raises(RuntimeError, match="site 5"):
        G.check_gemm_errors()
    y = G.gemm(x, w)
    G.check_gemm_errors()
    assert torch.allclose(y.float(), x.float() @ w.float().t(), rtol=2e-2, atol=2e-1)
