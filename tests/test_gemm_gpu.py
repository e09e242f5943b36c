"""tcgen05 GEMM against a plain fp32 PyTorch reference of the same contraction."""
import pytest
import torch

from parameter_server_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


def ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    Bm = b.float().t() if b_mn else b.float()
    return A @ Bm.t()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 512), (1000, 200, 136), (8192, 1024, 480)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(M + N + K)
    pad = lambda v: (v + 7) // 8 * 8
    a = torch.randn((K, pad(M)) if a_mn else (M, pad(K)), device="cuda").bfloat16()
    b = torch.randn((K, pad(N)) if b_mn else (N, pad(K)), device="cuda").bfloat16()
    av = a[:, :M] if a_mn else a[:, :K]
    bv = b[:, :N] if b_mn else b[:, :K]
    out = G.gemm(av, bv, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, M=M, N=N, K=K)
    G.check_gemm_errors()
    r = ref(av, bv, a_mn, b_mn)
    err = (out - r).abs().max().item()
    assert err <= 1e-2 * (K ** 0.5), f"max abs err {err}"
    assert torch.allclose(out, r, rtol=2e-2, atol=2e-2 * (K ** 0.5))


def test_epilogue_bias_relu_mask_accumulate():
    torch.manual_seed(0)
    M, N, K = 512, 256, 192
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda")
    y = G.linear_fwd(x, w, bias=bias, relu=True)
    r = torch.relu(x.float() @ w.float().t() + bias)
    assert torch.allclose(y.float(), r, rtol=2e-2, atol=2e-2)
    dy = torch.randn(M, N, device="cuda").bfloat16()
    mask = torch.randn(M, K, device="cuda").bfloat16()
    dx = G.linear_dgrad(dy, w, mask=mask)
    rdx = (dy.float() @ w.float()) * (mask.float() > 0)
    assert torch.allclose(dx.float(), rdx, rtol=2e-2, atol=5e-2)
    dw = torch.ones(N, K, device="cuda")
    G.linear_wgrad(dy, x, out=dw, accumulate=True)
    rdw = dy.float().t() @ x.float() + 1.0
    assert torch.allclose(dw, rdw, rtol=2e-2, atol=0.5)
    G.check_gemm_errors()


def test_grouped_wgrad_and_bias_grads_match_fp32_reference():
    """Several weight gradients in one persistent launch (wide group + narrow group) and all bias gradients in one."""
    torch.manual_seed(5)
    M = 2048
    shapes = [(1024, 480), (512, 1024), (256, 512), (128, 256), (512, 16), (64, 72)]   # (N_out, K_in)
    items, refs, bitems, brefs = [], [], [], []
    for n_out, k_in in shapes:
        ld = (k_in + 7) // 8 * 8
        dy = (torch.randn(M, n_out, device="cuda") * 0.5).bfloat16()
        xfull = (torch.randn(M, ld, device="cuda") * 0.5).bfloat16()
        x = xfull[:, :k_in]
        out = torch.zeros(n_out, k_in, device="cuda")
        items.append((dy, x, out))
        refs.append(dy.float().t() @ x.float())
        db = torch.zeros(n_out, device="cuda")
        bitems.append((dy, db))
        brefs.append(dy.float().sum(0))
    G.grouped_wgrad(items)
    G.bias_grads(bitems)
    G.check_gemm_errors()
    for (_, _, out), ref in zip(items, refs):
        assert torch.allclose(out, ref, rtol=2e-3, atol=2e-2), (out - ref).abs().max()
    for (_, db), ref in zip(bitems, brefs):
        assert torch.allclose(db, ref, rtol=1e-3, atol=1e-2)
    # explicit split and a second call accumulating on top (the outputs are not re-zeroed)
    G.grouped_wgrad(items[:3], split_k=3)
    G.check_gemm_errors()
    for (_, _, out), ref in zip(items[:3], refs[:3]):
        assert torch.allclose(out, 2 * ref, rtol=2e-3, atol=4e-2)


@pytest.mark.parametrize("M,dims", [(8192, (480, 1024, 1024, 512, 256)), (1000, (16, 512, 256, 128)), (300, (64, 256))])
def test_chained_mlp_forward_equals_layer_by_layer(M, dims):
    """All layers of an MLP in one persistent launch (a layer starts on a row block once the previous layer has stored
    it) must give bit for bit what one launch per layer gives: same tiles, same accumulation order."""
    torch.manual_seed(len(dims))
    ws = [(torch.randn(dims[i + 1], dims[i], device="cuda") * (2.0 / dims[i]) ** 0.5).bfloat16() for i in range(len(dims) - 1)]
    bs = [(torch.randn(dims[i + 1], device="cuda") * 0.1).bfloat16() for i in range(len(dims) - 1)]
    x = torch.randn(M, dims[0], device="cuda").bfloat16()
    one = [torch.empty(M, d, device="cuda", dtype=torch.bfloat16) for d in dims[1:]]
    two = [torch.empty(M, d, device="cuda", dtype=torch.bfloat16) for d in dims[1:]]
    a = x
    for w, b, o in zip(ws, bs, one):
        G.gemm(a, w, bias=b, relu=True, out=o)
        a = o
    layers, a = [], x
    for w, b, o in zip(ws, bs, two):
        layers.append(dict(a=a, w=w, bias=b, relu=True, out=o))
        a = o
    for _ in range(3):                       # the scratch counters are re-armed by every call
        for o in two:
            o.zero_()
        G.chain(layers)
        G.check_gemm_errors()
        for o1, o2 in zip(one, two):
            assert torch.equal(o1, o2)
    # and against the fp32 reference of the whole MLP
    r = x.float()
    for w, b in zip(ws, bs):
        r = torch.relu(r @ w.float().t() + b.float()).bfloat16().float()
    assert torch.allclose(two[-1].float(), r, rtol=5e-2, atol=5e-2)


def test_chained_dgrad_equals_layer_by_layer():
    torch.manual_seed(11)
    M, dims = 4096, (256, 512, 1024, 480)     # dz widths walking down an MLP: dz_i [M, dims[i]] -> dz_{i+1} [M, dims[i+1]]
    ws = [(torch.randn(dims[i], dims[i + 1], device="cuda") * 0.05).bfloat16() for i in range(len(dims) - 1)]   # [k][n]
    masks = [torch.randn(M, dims[i + 1], device="cuda").bfloat16() for i in range(len(dims) - 2)] + [None]
    dz = torch.randn(M, dims[0], device="cuda").bfloat16()
    one = [torch.empty(M, d, device="cuda", dtype=torch.bfloat16) for d in dims[1:]]
    two = [torch.zeros(M, d, device="cuda", dtype=torch.bfloat16) for d in dims[1:]]
    a = dz
    for w, m, o in zip(ws, masks, one):
        G.linear_dgrad(a, w, mask=m, out=o)
        a = o
    layers, a = [], dz
    for w, m, o in zip(ws, masks, two):
        layers.append(dict(a=a, w=w, mask=m, out=o))
        a = o
    G.chain(layers, b_mn=True)
    G.check_gemm_errors()
    for o1, o2 in zip(one, two):
        assert torch.equal(o1, o2)
