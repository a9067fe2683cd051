"""Caller integration on the GPU: MoELayer as the FFN of a small transformer (the shape of use in the
reference's examples/full_integration.py), trained for a few steps, and run under torch.compile."""

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

import flashfusedmoe_b200 as ffm  # noqa: E402
from flashfusedmoe_b200 import ops  # noqa: E402


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


class Block(nn.Module):
    def __init__(self, d_model, n_heads, ffn_dim, num_experts, top_k):
        super().__init__()
        self.n_heads = n_heads
        self.norm1 = nn.LayerNorm(d_model)
        self.qkv = nn.Linear(d_model, 3 * d_model, bias=False)
        self.proj = nn.Linear(d_model, d_model, bias=False)
        self.norm2 = nn.LayerNorm(d_model)
        self.moe = ffm.MoELayer(d_model, ffn_dim, num_experts, top_k, num_shared_experts=1, aux_loss_coeff=0.01,
                                z_loss_coeff=0.001)

    def forward(self, x):
        B, S, D = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(B, S, 3, self.n_heads, D // self.n_heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, D)
        x = x + self.proj(a)
        y, losses = self.moe(self.norm2(x))
        return x + y, losses["aux_loss"] + losses["z_loss"]


class TinyLM(nn.Module):
    def __init__(self, vocab=64, d_model=128, n_layers=2):
        super().__init__()
        self.emb = nn.Embedding(vocab, d_model)
        self.blocks = nn.ModuleList([Block(d_model, 4, 256, 8, 2) for _ in range(n_layers)])
        self.head = nn.Linear(d_model, vocab, bias=False)

    def forward(self, tokens):
        x = self.emb(tokens)
        extra = 0.0
        for b in self.blocks:
            x, l = b(x)
            extra = extra + l
        return self.head(x), extra


def _batch(step, vocab=64, B=8, S=64):
    g = torch.Generator().manual_seed(100 + step)
    start = torch.randint(0, vocab, (B, 1), generator=g)
    stride = torch.randint(1, 4, (B, 1), generator=g)
    seq = (start + stride * torch.arange(S + 1).unsqueeze(0)) % vocab   # arithmetic sequences: learnable
    return seq[:, :-1].cuda(), seq[:, 1:].cuda()


def test_transformer_with_moe_layers_trains():
    torch.manual_seed(0)
    model = TinyLM().cuda().bfloat16()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    first = last = None
    for step in range(40):
        x, y = _batch(step)
        logits, extra = model(x)
        ce = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), y.reshape(-1))
        loss = ce + extra.float()
        opt.zero_grad(set_to_none=True)
        loss.backward()
        for n, prm in model.named_parameters():
            assert prm.grad is not None and torch.isfinite(prm.grad).all(), n
        opt.step()
        first = float(ce.detach()) if first is None else first
        last = float(ce.detach())
    ops.check_status()
    assert last < 0.7 * first, (first, last)


def test_moe_layer_under_torch_compile_matches_eager():
    """fused_moe is excluded from tracing (torch.compiler.disable), so a compiled caller breaks the graph around it
    and must reproduce the eager results."""
    torch.manual_seed(1)
    model = TinyLM(n_layers=1).cuda().bfloat16()
    x, y = _batch(0)
    compiled = torch.compile(model, backend="aot_eager")

    def run(m):
        m.zero_grad(set_to_none=True)
        logits, extra = m(x)
        loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), y.reshape(-1)) + extra.float()
        loss.backward()
        return logits.detach().clone(), {n: p.grad.detach().clone() for n, p in model.named_parameters()}

    l0, g0 = run(model)
    l1, g1 = run(compiled)
    ops.check_status()
    # (not bit-exact: the attention backward around the layer accumulates with atomics)
    assert rel(l1, l0) <= 1e-2
    for n in g0:
        assert rel(g1[n], g0[n]) <= 2e-2, n
