"""GPU parity of the public API against the CPU oracle and the reference's golden vectors.

Tolerances: expert assignments and per-expert counts bit-exact; outputs, losses and gradients within
max|a - b| / max|b| <= 2e-2 (bf16 storage, fp32 accumulation), the bound BASELINE states.
"""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu

import flashfusedmoe_b200 as ffm  # noqa: E402
from flashfusedmoe_b200 import ops  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

DEV = "cuda"
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 2e-2


def rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def make_inputs(seed, N, D, E, F, scale=0.02, dtype=torch.bfloat16):
    torch.manual_seed(seed)
    h = torch.randn(N, D).to(dtype)
    g = (torch.randn(E, D) * scale).to(dtype)
    wu = (torch.randn(E, F, D) * scale).to(dtype)
    wd = (torch.randn(E, D, F // 2) * scale).to(dtype)
    go = torch.randn(N, D).to(dtype)
    return h, g, wu, wd, go


def run_ours(h, g, wu, wd, go, k, **kw):
    hd, gd, wud, wdd = [t.to(DEV).requires_grad_() for t in (h, g, wu, wd)]
    out, losses = ffm.fused_moe(hd, gd, wud, wdd, top_k=k, return_metrics=True, **kw)
    loss = (out.float() * go.to(DEV).float()).sum()
    for n in ("aux_loss", "z_loss"):
        if n in losses:
            loss = loss + losses[n]
    loss.backward()
    ops.check_status()
    return out, losses, (hd.grad, gd.grad, wud.grad, wdd.grad)


def compare_with_oracle(h, g, wu, wd, go, k, activation, gating, aux, z, tol=TOL):
    out, losses, grads = run_ours(h, g, wu, wd, go, k, activation=activation, gating=gating, aux_loss_coeff=aux,
                                  z_loss_coeff=z)
    fw = orc.fused_moe_forward(h, g, wu, wd, k, activation, gating, aux, z, dtype=torch.bfloat16)
    bw = orc.fused_moe_backward(fw, go)
    E = g.shape[0]
    counts = torch.bincount(fw["topk_idx"].reshape(-1), minlength=E)
    assert torch.equal(losses["tokens_per_expert"].cpu().long(), counts), "per-expert counts must be bit-exact"
    assert rel(out, fw["out"]) <= tol
    for name, ours in zip(("dH", "dGate", "dW_up", "dW_down"), grads):
        assert rel(ours, bw[name]) <= tol, name
    for n in ("aux_loss", "z_loss"):
        if n in fw["losses"]:
            ref = float(fw["losses"][n])
            assert abs(float(losses[n]) - ref) <= 1e-3 * abs(ref) + 1e-7, n
    return fw


@pytest.mark.parametrize("activation,gating,aux,z", [("swiglu", "softmax", 0.01, 0.001), ("geglu", "softmax", 0.0, 0.0),
                                                     ("relu_squared", "sigmoid", 0.01, 0.001),
                                                     ("swiglu", "sigmoid", 0.0, 0.0)])
def test_small_layer_vs_oracle(activation, gating, aux, z):
    h, g, wu, wd, go = make_inputs(21, 96, 64, 8, 128, scale=0.1)
    compare_with_oracle(h, g, wu, wd, go, 2, activation, gating, aux, z)


@pytest.mark.parametrize("N,D,E,F,k", [(1, 64, 4, 128, 1), (3, 64, 16, 128, 4), (50, 128, 64, 128, 8),
                                       (200, 64, 8, 256, 3), (512, 256, 8, 1024, 2), (130, 192, 24, 384, 2)])
def test_shapes_vs_oracle(N, D, E, F, k):
    # includes N=1, E > N (empty experts), top_k 1/3/4/8 and BASELINE configs[0]'s shape
    h, g, wu, wd, go = make_inputs(N + E, N, D, E, F, scale=0.05)
    compare_with_oracle(h, g, wu, wd, go, k, "swiglu", "softmax", 0.01, 0.001)


def test_routing_bit_exact_vs_oracle_on_identical_logits():
    """Indices, their order and per-expert counts equal the reference rule applied to the kernel's own logits;
    the kernel's bf16 logits equal the oracle's up to one unit in the last place."""
    for seed, (N, D, E, k) in enumerate([(2048, 256, 8, 2), (512, 512, 64, 6), (128, 1024, 256, 8)]):
        h, g, _, _, _ = make_inputs(seed, N, D, E, 64, scale=0.02)
        r = ops.route_forward(h.to(DEV), g.to(DEV), k, "softmax")
        lg = r.logits.cpu()
        w_o, i_o = orc.route(lg, "softmax", k)
        assert torch.equal(r.topk_idx.cpu().long(), i_o)
        assert torch.allclose(r.topk_w.cpu(), w_o, atol=2e-6, rtol=1e-4)
        ref_lg = orc.gate_logits(h, g, torch.bfloat16)
        # one bf16 unit in the last place, plus the fp32 accumulation-order error of a D-term dot product
        # (it dominates for logits that cancel to nearly zero)
        diff = (lg.float() - ref_lg.float()).abs()
        ulp = torch.maximum(lg.float().abs(), ref_lg.float().abs()) * 2.0 ** -7
        # (E > 32 runs the gate GEMM on the tensor cores, whose fp32 accumulation truncates: wider allowance)
        acc_err = (2e-6 if E <= 32 else 1.5e-5) * (h.float().abs() @ g.float().abs().T)
        assert (diff <= ulp + acc_err).all(), float((diff / (ulp + acc_err)).max())
        same_rows = (lg == ref_lg).all(1)
        _, i_ref = orc.route(ref_lg, "softmax", k)
        assert torch.equal(i_o[same_rows], i_ref[same_rows])
        assert same_rows.float().mean() > (0.9 if E <= 32 else 0.5), float(same_rows.float().mean())


def test_golden_reference_outputs_bf16():
    """The unmodified reference's own outputs on bf16 inputs (recorded on CPU) vs the CUDA path."""
    gold = torch.load(os.path.join(GOLD, "layer_small_bf16.pt"))
    N, D, E, F, k = gold["shape"]
    i = gold["inputs"]
    for key, case in gold["cases"].items():
        activation, gating, aux, z = key.split("/")
        out, losses, grads = run_ours(i["h"], i["g"], i["wu"], i["wd"], i["go"], k, activation=activation,
                                      gating=gating, aux_loss_coeff=float(aux), z_loss_coeff=float(z))
        assert torch.equal(losses["tokens_per_expert"].cpu(), case["tokens_per_expert"]), key
        assert rel(out, case["out"]) <= TOL, key
        for name, ours in zip(("dH", "dGate", "dW_up", "dW_down"), grads):
            assert rel(ours, case[name]) <= TOL, (key, name)
        for n, v in case["losses"].items():
            assert abs(float(losses[n]) - v) <= 2e-3 * abs(v) + 1e-7, (key, n)


def test_config1_fp32_inputs_under_autocast():
    """BASELINE configs[0] (fp32 tensors): runs under bf16 autocast; compared with the bf16 oracle."""
    h, g, wu, wd, go = make_inputs(0, 512, 256, 8, 1024, dtype=torch.float32)
    hd, gd, wud, wdd = [t.to(DEV).requires_grad_() for t in (h, g, wu, wd)]
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out, losses = ffm.fused_moe(hd, gd, wud, wdd, top_k=2, aux_loss_coeff=0.01, z_loss_coeff=0.001,
                                    return_metrics=True)
    (out.float() * go.to(DEV)).sum().backward()
    assert hd.grad.dtype == torch.float32 and wud.grad.dtype == torch.float32
    fw = orc.fused_moe_forward(h, g, wu, wd, 2, "swiglu", "softmax", 0.01, 0.001, dtype=torch.bfloat16)
    bw = orc.fused_moe_backward(fw, go, grad_aux=0.0, grad_z=0.0)
    assert torch.equal(losses["tokens_per_expert"].cpu().long(), torch.bincount(fw["topk_idx"].reshape(-1), minlength=8))
    assert rel(out, fw["out"]) <= TOL
    assert rel(hd.grad, bw["dH"]) <= TOL and rel(wdd.grad, bw["dW_down"]) <= TOL
    with pytest.raises(NotImplementedError, match="bfloat16"):
        ffm.fused_moe(hd, gd, wud, wdd, top_k=2)


def test_aux_loss_grad_modes():
    h, g, wu, wd, go = make_inputs(5, 128, 64, 8, 128, scale=0.1)
    _, _, grads_a = run_ours(h, g, wu, wd, go * 0, 2, aux_loss_coeff=0.5)
    assert grads_a[1].abs().max() > 0, "analytic aux loss reaches the gate"
    ffm.set_aux_loss_grad("reference_cuda")
    try:
        _, _, grads_c = run_ours(h, g, wu, wd, go * 0, 2, aux_loss_coeff=0.5)
    finally:
        ffm.set_aux_loss_grad("analytic")
    assert grads_c[1].abs().max() == 0, "softmax-gating aux loss is a constant on the reference's CUDA path"


def test_recompute_is_bit_identical():
    # reference tests/test_production.py:258-311 (atol=0)
    h, g, wu, wd, go = make_inputs(9, 300, 128, 8, 256, scale=0.05)
    o1, _, g1 = run_ours(h, g, wu, wd, go, 2, recompute_activations=False)
    o2, _, g2 = run_ours(h, g, wu, wd, go, 2, recompute_activations=True)
    assert torch.equal(o1, o2)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)


def test_deterministic_and_expanded_grad_output():
    h, g, wu, wd, go = make_inputs(10, 256, 64, 8, 128, scale=0.05)
    o1, _, g1 = run_ours(h, g, wu, wd, go, 2)
    o2, _, g2 = run_ours(h, g, wu, wd, go, 2)
    assert torch.equal(o1, o2) and all(torch.equal(a, b) for a, b in zip(g1, g2))
    hd = h.to(DEV).requires_grad_()
    out, _ = ffm.fused_moe(hd, g.to(DEV), wu.to(DEV), wd.to(DEV), top_k=2)
    out.sum().backward()  # stride-0 expanded grad_output: must be densified, not read as garbage
    assert torch.isfinite(hd.grad).all()
    _, _, g3 = run_ours(h, g, wu, wd, torch.ones_like(go), 2)
    assert torch.equal(hd.grad, g3[0])


def test_overflow_error_and_metrics():
    h, g, wu, wd, go = make_inputs(12, 256, 64, 8, 128, scale=0.05)
    args = [t.to(DEV) for t in (h, g, wu, wd)]
    with pytest.raises(RuntimeError, match="MoE routing overflow"):
        ffm.fused_moe(*args, top_k=2, max_tokens_per_expert=1, allow_dropped_tokens=False)
    out, losses = ffm.fused_moe(*args, top_k=2, max_tokens_per_expert=1, allow_dropped_tokens=True, return_metrics=True)
    assert set(losses) == {"tokens_per_expert", "max_expert_load", "min_expert_load", "expert_load_imbalance"}
    assert int(losses["tokens_per_expert"].sum()) == 256 * 2
    assert int(losses["max_expert_load"]) == int(losses["tokens_per_expert"].max())


def test_expert_bias_and_scoring_factor():
    h, g, wu, wd, go = make_inputs(13, 200, 64, 8, 128, scale=0.05)
    bias = torch.linspace(-0.5, 0.5, 8)
    out, losses = ffm.fused_moe(h.to(DEV), g.to(DEV), wu.to(DEV), wd.to(DEV), top_k=2, expert_bias=bias.to(DEV),
                                scoring_factor=2.5, return_metrics=True)
    lg = orc.gate_logits(h, g, torch.bfloat16)
    w, idx = orc.route(lg, "softmax", 2, expert_bias=bias, scoring_factor=2.5)
    assert torch.equal(losses["tokens_per_expert"].cpu().long(), torch.bincount(idx.reshape(-1), minlength=8))


@pytest.mark.parametrize("activation", ["swiglu", "geglu"])
def test_moe_layer_with_shared_expert_vs_oracle(activation):
    torch.manual_seed(3)
    layer = ffm.MoELayer(128, 256, 8, 2, activation=activation, num_shared_experts=1, aux_loss_coeff=0.01).to(DEV).bfloat16()
    x = torch.randn(4, 50, 128, device=DEV).bfloat16().requires_grad_()
    y, losses = layer(x)
    assert y.shape == x.shape and "aux_loss" in losses
    go = torch.randn_like(y)
    (y.float() * go.float()).sum().backward()
    ops.check_status()
    p = {n: t.detach().cpu() for n, t in layer.named_parameters()}
    xf = x.detach().cpu().reshape(-1, 128)
    fw = orc.fused_moe_forward(xf, p["gate.weight"], p["w_up"], p["w_down"], 2, activation, "softmax", 0.01, 0.0,
                               dtype=torch.bfloat16)
    sh_act = "geglu_erf" if activation == "geglu" else activation
    shared = orc.glu_ffn(xf, p["shared_expert.w_gate.weight"], p["shared_expert.w_up.weight"],
                         p["shared_expert.w_down.weight"], sh_act, torch.bfloat16)
    ref = (fw["out"].float() + shared.float()).to(torch.bfloat16)
    assert rel(y.reshape(-1, 128), ref) <= TOL
    # shared-expert gradients against autograd of the same restatement
    ws = [p[f"shared_expert.{n}.weight"].float().requires_grad_() for n in ("w_gate", "w_up", "w_down")]
    xs = xf.float().requires_grad_()
    gate_o, up_o = xs @ ws[0].T, xs @ ws[1].T
    a = torch.nn.functional.silu(gate_o) if activation == "swiglu" else torch.nn.functional.gelu(gate_o)
    ((a * up_o) @ ws[2].T * go.cpu().float().reshape(-1, 128)).sum().backward()
    for n, w in zip(("w_gate", "w_up", "w_down"), ws):
        assert rel(getattr(layer.shared_expert, n).weight.grad, w.grad) <= TOL, n
    bw = orc.fused_moe_backward(fw, go.cpu().reshape(-1, 128), grad_aux=0.0)
    assert rel(x.grad.reshape(-1, 128), bw["dH"].float() + xs.grad) <= TOL


def test_single_gpu_benchmark_shape_properties():
    """BASELINE configs[1] shape (16,384 tokens, D=1024, ffn 4096, E=8, k=2): size-independent properties and a
    per-expert torch fp32 check on the GPU."""
    torch.manual_seed(1)
    N, D, F, E, k = 16384, 1024, 4096, 8, 2
    H = F // 2
    h = torch.randn(N, D, device=DEV).bfloat16().requires_grad_()
    g = (torch.randn(E, D, device=DEV) * 0.02).bfloat16().requires_grad_()
    wu = (torch.randn(E, F, D, device=DEV) * 0.02).bfloat16().requires_grad_()
    wd = (torch.randn(E, D, H, device=DEV) * 0.02).bfloat16().requires_grad_()
    out, losses = ffm.fused_moe(h, g, wu, wd, top_k=k, return_metrics=True)
    go = torch.randn_like(out)
    out.backward(go)
    ops.check_status()
    assert int(losses["tokens_per_expert"].sum()) == N * k
    assert torch.isfinite(out).all() and all(torch.isfinite(t.grad).all() for t in (h, g, wu, wd))
    # torch restatement on the GPU from the kernel's own routing
    r = ops.route_forward(h.detach(), g.detach(), k, "softmax")
    idx, w = r.topk_idx.long(), r.topk_w.bfloat16().float()
    ref = torch.zeros(N, D, device=DEV)
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        x = h.detach()[tok]
        pre = (x.float() @ wu.detach()[e].float().T).bfloat16().float()
        a = (torch.nn.functional.silu(pre[:, :H]) * pre[:, H:]).bfloat16()
        y = (a.float() @ wd.detach()[e].float().T).bfloat16().float()
        ref.index_add_(0, tok, y * w[tok, slot].unsqueeze(-1))
    assert rel(out, ref) <= TOL
    # linearity of the backward in grad_output
    h2 = h.detach().clone().requires_grad_()
    out2, _ = ffm.fused_moe(h2, g.detach(), wu.detach(), wd.detach(), top_k=k)
    out2.backward(2 * go)
    assert rel(h2.grad, 2 * h.grad.float()) <= 1e-2
