"""GPU: the BASELINE configurations beyond configs[1] at their full single-GPU shapes.

Sizes here are too large for the CPU oracle, so each case checks (a) routing decisions against the oracle's rule on
the kernel's own logits, (b) the output and the input gradient of a sample of tokens against a torch fp32 autograd
restatement on the GPU (a token's output and dH depend only on that token), (c) size-independent properties:
token conservation, finiteness, determinism.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

import flashfusedmoe_b200 as ffm  # noqa: E402
from flashfusedmoe_b200 import ops  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

DEV = "cuda"
TOL = 2e-2


def rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def sample_reference(h, g, wu, wd, go, idx, sample, k, gating="softmax", shared=None):
    """fp32 autograd restatement for the sampled tokens, using the kernel's expert choice `idx`."""
    H = wu.shape[1] // 2
    x = h[sample].float().requires_grad_()
    logits = (x @ g.float().T).bfloat16().float() + 0.0 * x.sum()  # value rounded like the kernel's, graph kept below
    logits = x @ g.float().T + (logits - x @ g.float().T).detach()
    sel = idx[sample].long()
    if gating == "softmax":
        w = torch.softmax(logits.gather(1, sel), -1)
    else:
        sc = torch.sigmoid(logits).gather(1, sel)
        w = sc / (sc.sum(-1, keepdim=True) + 1e-6)
    w = w + (w.bfloat16().float() - w).detach()
    out = torch.zeros(len(sample), h.shape[1], device=h.device)
    for i in range(len(sample)):
        for j in range(k):
            e = int(sel[i, j])
            pre = x[i] @ wu[e].float().T
            a = torch.nn.functional.silu(pre[:H]) * pre[H:]
            out[i] = out[i] + w[i, j] * (a @ wd[e].float().T)
    if shared is not None:
        sg, su, sd = [t.float() for t in shared]
        out = out + (torch.nn.functional.silu(x @ sg.T) * (x @ su.T)) @ sd.T
    (out * go[sample].float()).sum().backward()
    return out.detach(), x.grad


def run_case(N, D, F, E, k, seed, bias=None, shared_ffn=None, backward=True, sample_n=24):
    torch.manual_seed(seed)
    H = F // 2
    h = torch.randn(N, D, device=DEV).bfloat16().requires_grad_(backward)
    g = (torch.randn(E, D, device=DEV) * 0.02).bfloat16()
    wu = (torch.randn(E, F, D, device=DEV) * 0.02).bfloat16().requires_grad_(backward)
    wd = (torch.randn(E, D, H, device=DEV) * 0.02).bfloat16().requires_grad_(backward)
    go = torch.randn(N, D, device=DEV).bfloat16()
    out, losses = ffm.fused_moe(h, g, wu, wd, top_k=k, expert_bias=bias, return_metrics=True)
    assert int(losses["tokens_per_expert"].sum()) == N * k
    assert torch.isfinite(out).all()
    r = ops.route_forward(h.detach(), g, k, "softmax", bias)
    _, i_o = orc.route(r.logits.cpu(), "softmax", k, None if bias is None else bias.cpu())
    assert torch.equal(r.topk_idx.cpu().long(), i_o), "expert assignment differs from the rule"
    assert torch.equal(losses["tokens_per_expert"].cpu().long(), torch.bincount(i_o.reshape(-1), minlength=E))
    sample = torch.randperm(N, device=DEV)[:sample_n]
    if backward:
        out.backward(go)
        ops.check_status()
        assert all(torch.isfinite(t.grad).all() for t in (h, wu, wd))
        ref_out, ref_dh = sample_reference(h.detach(), g, wu.detach(), wd.detach(), go, r.topk_idx, sample, k)
        assert rel(out[sample], ref_out) <= TOL
        assert rel(h.grad[sample], ref_dh) <= 3e-2
        # determinism of the whole step
        h2 = h.detach().clone().requires_grad_()
        wu2, wd2 = wu.detach().clone().requires_grad_(), wd.detach().clone().requires_grad_()
        out2, _ = ffm.fused_moe(h2, g, wu2, wd2, top_k=k, expert_bias=bias)
        out2.backward(go)
        assert torch.equal(out, out2) and torch.equal(h.grad, h2.grad) and torch.equal(wd.grad, wd2.grad)
    else:
        ops.check_status()
        with torch.enable_grad():
            ref_out, _ = sample_reference(h.detach(), g, wu.detach(), wd.detach(), go, r.topk_idx, sample, k)
        assert rel(out[sample], ref_out) <= TOL
    return losses


def test_config3_mixtral_shape_with_zipf_bias():
    """configs[2]: D=4096, E=8, top-2, ffn_dim 2 x 14336, 8192 tokens, Zipf(s=1.1) gate bias (log-probabilities over a
    seeded permutation of the experts) for load imbalance; forward + backward at EP = 1."""
    E = 8
    g = torch.Generator().manual_seed(2)
    perm = torch.randperm(E, generator=g)
    p = 1.0 / torch.arange(1, E + 1).float() ** 1.1
    bias = torch.log(p / p.sum())[perm].to(DEV)
    losses = run_case(8192, 4096, 28672, E, 2, seed=2, bias=bias)
    tpe = losses["tokens_per_expert"].float()
    assert tpe.max() / tpe.mean() > 1.5, "the bias must produce a visibly imbalanced load"


def test_config4_fine_grained_shape():
    """configs[3] local shape: D=2048, 64 experts, top-6, ffn_dim 2 x 1408, 16,384 tokens."""
    run_case(16384, 2048, 2816, 64, 6, seed=3)


def test_config4_layer_with_merged_shared_experts_vs_oracle():
    """configs[3] layer (2 shared experts merged into one FFN of ffn_dim 2 x 2816) on a 1024-token slice vs the oracle."""
    torch.manual_seed(3)
    layer = ffm.MoELayer(2048, 2816, 64, 6, num_shared_experts=2, shared_ffn_dim=2 * 2816).to(DEV).bfloat16()
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0.0, 0.02)
    x = torch.randn(1024, 2048, device=DEV).bfloat16()
    y, _ = layer(x)
    p = {n: t.detach().cpu() for n, t in layer.named_parameters()}
    fw = orc.fused_moe_forward(x.cpu(), p["gate.weight"], p["w_up"], p["w_down"], 6, dtype=torch.bfloat16)
    shared = orc.glu_ffn(x.cpu(), p["shared_expert.w_gate.weight"], p["shared_expert.w_up.weight"],
                         p["shared_expert.w_down.weight"], "swiglu", torch.bfloat16)
    assert rel(y.cpu(), fw["out"].float() + shared.float()) <= TOL


def test_config5_decode_shape_forward_only():
    """configs[4]: D=7168, 256 experts, top-8, ffn_dim 2 x 2048, 128 tokens, forward only."""
    with torch.no_grad():
        run_case(128, 7168, 4096, 256, 8, seed=4, backward=False, sample_n=8)
