"""DLRM end to end on one GPU: the hand-written forward matches a plain fp32 PyTorch restatement,
training reduces the loss, and the model kernels match their references."""
import pytest
import torch

from parameter_server_b200 import C
from parameter_server_b200.models import DLRM, DLRMConfig, SyntheticCTR

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,F,emb_bf16", [(128, 26, False), (128, 26, True), (64, 9, False), (64, 9, True)])
def test_interaction_kernels_match_reference(D, F, emb_bf16):
    """fp32 PyTorch reference of the same op; the kernels stage their operands as bf16, hence the tolerances. With
    bf16 embedding rows (what a bf16 pull delivers) the result must equal the fp32-input run bit for bit, because the
    fp32 path rounds the rows to bf16 the same way."""
    torch.manual_seed(0)
    B = 300
    npairs = (F + 1) * F // 2
    ldo = (D + npairs + 7) // 8 * 8
    bottom = torch.randn(B, D, device="cuda").bfloat16()
    emb = torch.randn(B, F, D, device="cuda") * 0.1
    emb_in = emb.bfloat16() if emb_bf16 else emb
    out = torch.empty(B, ldo, device="cuda", dtype=torch.bfloat16)
    assert C.interaction_fwd(bottom.data_ptr(), D, emb_in.data_ptr(), F, D, out.data_ptr(), ldo, B, 0, emb_bf16) == 0
    T = torch.cat([bottom.float()[:, None], emb], 1)
    Z = torch.bmm(T, T.transpose(1, 2))
    ii, jj = torch.tril_indices(F + 1, F + 1, offset=-1)
    ref = torch.cat([bottom.float(), Z[:, ii, jj], torch.zeros(B, ldo - D - npairs, device="cuda")], 1)
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    # backward against autograd
    Tg = T.clone().requires_grad_(True)
    Zg = torch.bmm(Tg, Tg.transpose(1, 2))
    o = torch.cat([Tg[:, 0], Zg[:, ii, jj]], 1)
    dout = torch.randn(B, ldo, device="cuda").bfloat16()
    o.backward(dout.float()[:, :o.shape[1]])
    dbot = torch.empty(B, D, device="cuda", dtype=torch.bfloat16)
    demb = torch.empty(B, F, D, device="cuda")
    assert C.interaction_bwd(dout.data_ptr(), ldo, bottom.data_ptr(), D, emb_in.data_ptr(), F, D, dbot.data_ptr(), D,
                             demb.data_ptr(), B, False, 0, emb_bf16) == 0
    assert torch.allclose(demb, Tg.grad[:, 1:], rtol=2e-2, atol=1e-2)  # operands are staged as bf16
    assert torch.allclose(dbot.float(), Tg.grad[:, 0], rtol=2e-2, atol=5e-2)
    if emb_bf16:
        out32 = torch.empty_like(out)
        demb32 = torch.empty_like(demb)
        dbot32 = torch.empty_like(dbot)
        assert C.interaction_fwd(bottom.data_ptr(), D, emb.data_ptr(), F, D, out32.data_ptr(), ldo, B, 0, False) == 0
        assert C.interaction_bwd(dout.data_ptr(), ldo, bottom.data_ptr(), D, emb.data_ptr(), F, D, dbot32.data_ptr(), D,
                                 demb32.data_ptr(), B, False, 0, False) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, out32) and torch.equal(demb, demb32) and torch.equal(dbot, dbot32)
    # relu mask on the bottom gradient
    dbot_m = torch.empty_like(dbot)
    assert C.interaction_bwd(dout.data_ptr(), ldo, bottom.data_ptr(), D, emb_in.data_ptr(), F, D, dbot_m.data_ptr(), D,
                             demb.data_ptr(), B, True, 0, emb_bf16) == 0
    torch.cuda.synchronize()
    assert torch.equal(dbot_m, torch.where(bottom > 0, dbot, torch.zeros_like(dbot)))


def test_bce_head_and_bias_grad():
    torch.manual_seed(1)
    B, K = 1000, 256
    h = torch.relu(torch.randn(B, K, device="cuda")).bfloat16()
    w = (torch.randn(K, device="cuda") * 0.1).bfloat16()
    b = torch.tensor([0.3], device="cuda").bfloat16()
    y = (torch.rand(B, device="cuda") < 0.3).float()
    loss = torch.zeros(1, device="cuda")
    dz = torch.empty(B, K, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(K, device="cuda")
    db = torch.zeros(1, device="cuda")
    assert C.bce_head(h.data_ptr(), K, w.data_ptr(), b.data_ptr(), y.data_ptr(), B, K, 1.0 / B, loss.data_ptr(), 0,
                      dz.data_ptr(), K, dw.data_ptr(), db.data_ptr(), 0) == 0
    hf = h.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    bf = b.float().requires_grad_(True)
    ref = torch.nn.functional.binary_cross_entropy_with_logits(hf @ wf + bf, y)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-4
    assert torch.allclose(dw, wf.grad, rtol=1e-3, atol=1e-5)
    assert torch.allclose(db, bf.grad, rtol=1e-3, atol=1e-6)
    assert torch.allclose(dz.float(), hf.grad * (h.float() > 0), rtol=2e-2, atol=1e-6)
    dbias = torch.zeros(K, device="cuda")
    assert C.bias_grad(dz.data_ptr(), K, B, K, dbias.data_ptr(), 0) == 0
    assert torch.allclose(dbias, dz.float().sum(0), rtol=1e-3, atol=1e-6)


def test_forward_matches_reference_and_loss_decreases():
    cfg = DLRMConfig(vocab_max=2e4)
    B = 1024
    model = DLRM(cfg, B, table_capacity=1 << 18)
    data = SyntheticCTR(cfg, B, pool=4, seed=5)
    batch = data.next()
    model.load_batch(*batch)
    ref = model.reference_loss()
    model.forward_backward()
    got = model.read_loss()
    model.check()
    assert abs(got - ref) < 2e-2 * max(1.0, abs(ref)), (got, ref)
    first = got
    for _ in range(60):
        model.train_step(*data.next())
    model.check()
    model.load_batch(*batch)
    later = model.reference_loss()
    assert later < first, (first, later)
    assert model.sparse.size() > 0


def test_graph_replay_matches_eager():
    """The same steps, launched eagerly and replayed from a CUDA graph, end in the same parameters."""
    cfg = DLRMConfig(vocab_max=2e4)
    B = 512

    def run(use_graph):
        model = DLRM(cfg, B, table_capacity=1 << 17, seed=3)
        data = SyntheticCTR(cfg, B, pool=3, seed=9)
        for _ in range(3):
            model.train_step(*data.next())
        if use_graph:
            model.enable_graph()
        losses = []
        for _ in range(6):
            model.train_step(*data.next())
            losses.append(model.read_loss())
        model.check()
        return losses, model.dense.flat_params.float().clone(), model.sparse.size()

    le, pe, ne = run(False)
    lg, pg, ng = run(True)
    assert ne == ng
    assert max(abs(a - b) for a, b in zip(le, lg)) < 5e-3, (le, lg)
    assert torch.allclose(pe, pg, rtol=0, atol=2e-2)


def test_overlapped_step_matches_the_serial_step():
    """The sparse pull / push on a side stream with a bounded CTA budget, beside the dense GEMMs, computes the same
    step as the serial launch order (up to the order of fp32 atomics in the gradient sums)."""
    cfg = DLRMConfig(vocab_max=2e4)
    B = 512

    def run(overlap, graph):
        model = DLRM(cfg, B, table_capacity=1 << 17, seed=3, overlap=overlap)
        data = SyntheticCTR(cfg, B, pool=3, seed=9)
        for _ in range(3):
            model.train_step(*data.next())
        if graph:
            model.enable_graph()
        losses = []
        for _ in range(6):
            model.train_step(*data.next())
            losses.append(model.read_loss())
        model.check()
        return losses, model.dense.flat_params.float().clone(), model.sparse.size()

    ls, ps_, ns = run(False, False)
    for graph in (False, True):
        lo, po, no = run(True, graph)
        assert no == ns
        assert max(abs(a - b) for a, b in zip(ls, lo)) < 5e-3, (ls, lo)
        assert torch.allclose(ps_, po, rtol=0, atol=2e-2)


def test_staged_batches_and_tail_overlap_match_the_plain_step():
    """``stage`` + ``train_step()`` (the next batch crosses PCIe while the queued step runs) and the arrangement used
    from three ranks on (sparse push beside the dense push, both as whole-SM CTAs on disjoint SMs) compute the same
    step as ``train_step(batch)`` on one stream."""
    cfg = DLRMConfig(vocab_max=2e4)
    B = 512

    def run(staged, tail, graph):
        model = DLRM(cfg, B, table_capacity=1 << 17, seed=3, overlap=False, tail_overlap=tail)
        assert model.tail_overlap == tail
        data = SyntheticCTR(cfg, B, pool=3, seed=9)
        for _ in range(3):
            model.train_step(*data.next())
        if graph:
            model.enable_graph()
        losses = []
        if staged:
            model.stage(*data.next())
            for i in range(6):
                model.train_step()
                if i + 1 < 6:
                    model.stage(*data.next())
                losses.append(model.read_loss())
        else:
            for _ in range(6):
                model.train_step(*data.next())
                losses.append(model.read_loss())
        model.check()
        return losses, model.dense.flat_params.float().clone(), model.sparse.size()

    ls, ps_, ns = run(False, False, False)
    for staged, tail, graph in ((True, False, True), (False, True, False), (True, True, True)):
        lo, po, no = run(staged, tail, graph)
        assert no == ns
        assert max(abs(a - b) for a, b in zip(ls, lo)) < 5e-3, (ls, lo)
        assert torch.allclose(ps_, po, rtol=0, atol=2e-2)
    with pytest.raises(RuntimeError):
        DLRM(cfg, B, table_capacity=1 << 17, seed=3, overlap=False).train_step()
