"""GPT on the dense parameter-server path: forward loss against a plain fp32 PyTorch restatement with the
same parameters, and a few optimizer steps that reduce the loss."""
import math

import pytest
import torch
import torch.nn.functional as F

from parameter_server_b200.models.gpt import GPT, GPTConfig

pytestmark = pytest.mark.gpu


def reference_loss(model, tokens, targets):
    cfg = model.cfg
    P = {k: v.detach().float() for k, v in model.main.params.items()}
    for i, t in enumerate(model.qkv):
        if t is not None:
            P[f"h{i}.qkv.w"] = t.params["w"].detach().float()
    B, T = tokens.shape
    x = P["wte"][tokens] + P["wpe"][:T]
    for i in range(cfg.n_layer):
        h = F.layer_norm(x, (cfg.d_model,), P[f"h{i}.ln1.g"], P[f"h{i}.ln1.b"])
        qkv = h @ P[f"h{i}.qkv.w"].t() + P[f"h{i}.qkv.b"]
        q, k, v = qkv.view(B, T, 3, cfg.n_head, -1).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, cfg.d_model)
        x = x + a @ P[f"h{i}.proj.w"].t() + P[f"h{i}.proj.b"]
        h = F.layer_norm(x, (cfg.d_model,), P[f"h{i}.ln2.g"], P[f"h{i}.ln2.b"])
        h = F.gelu(h @ P[f"h{i}.fc.w"].t() + P[f"h{i}.fc.b"], approximate="tanh")
        x = x + h @ P[f"h{i}.out.w"].t() + P[f"h{i}.out.b"]
    x = F.layer_norm(x, (cfg.d_model,), P["lnf.g"], P["lnf.b"])
    return F.cross_entropy((x @ P["wte"].t()).view(-1, cfg.vocab), targets.reshape(-1)).item()


def test_tiny_gpt_matches_reference_and_learns():
    cfg = GPTConfig(n_layer=2, d_model=256, n_head=4, d_ff=1024, vocab=512, seq_len=64, lr=3e-3, weight_decay=0.0)
    model = GPT(cfg, seed=1)
    gen = torch.Generator().manual_seed(0)
    data = torch.randint(0, cfg.vocab, (8, cfg.seq_len + 1), generator=gen).cuda()
    tokens, targets = data[:, :-1], data[:, 1:]
    ref = reference_loss(model, tokens, targets)
    _, loss = model.forward(tokens, targets)
    assert abs(loss.item() - ref) < 3e-2, (loss.item(), ref)
    assert abs(ref - math.log(cfg.vocab)) < 0.5
    first = None
    for step in range(12):
        l = model.train_step(tokens, targets, micro_batches=2).item()
        first = l if first is None else first
    model.check()
    assert l < first - 0.5, (first, l)
