"""CPU: the oracle (oracle/moe_oracle.py) replayed against the golden vectors that
oracle/pin_against_reference.py recorded from the unmodified reference."""

import os

import pytest
import torch

from oracle import moe_oracle as orc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def test_routing_rule_golden():
    gold = torch.load(os.path.join(GOLD, "routing_rule.pt"))
    assert len(gold) == 10
    for name, case in gold.items():
        w, idx = orc.route(case["logits"], case["gating"], case["k"])
        assert torch.equal(idx.to(torch.int32), case["idx"]), name
        assert torch.allclose(w, case["w"], atol=1e-6, rtol=1e-5), name


def test_lowest_index_wins_ties():
    lg = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0, 0.0, 2.0, 2.0], [0.0] * 8])
    _, idx = orc.route(lg, "softmax", 3)
    assert idx.tolist() == [[1, 2, 4], [0, 1, 2]]


@pytest.mark.parametrize("tag,tol", [("layer_small_fp32", 2e-5), ("layer_small_bf16", 2e-2)])
def test_layer_small_golden(tag, tol):
    gold = torch.load(os.path.join(GOLD, f"{tag}.pt"))
    N, D, E, F, k = gold["shape"]
    i = gold["inputs"]
    dtype = i["h"].dtype
    for key, case in gold["cases"].items():
        activation, gating, aux, z = key.split("/")
        fw = orc.fused_moe_forward(i["h"], i["g"], i["wu"], i["wd"], k, activation, gating, float(aux), float(z),
                                   dtype=dtype)
        bw = orc.fused_moe_backward(fw, i["go"])
        assert torch.equal(fw["topk_idx"].to(torch.int32), case["topk_idx"]), key
        assert torch.equal(torch.bincount(fw["topk_idx"].reshape(-1), minlength=E).to(torch.int32),
                           case["tokens_per_expert"]), key
        for name in ("out",):
            assert rel(fw[name], case[name]) <= tol, (key, name)
        for name in ("dH", "dGate", "dW_up", "dW_down"):
            assert rel(bw[name], case[name]) <= tol, (key, name)
        for name, v in case["losses"].items():
            assert abs(float(fw["losses"][name]) - v) <= 1e-5 * max(1.0, abs(v)), (key, name)


def test_config1_golden():
    """BASELINE configs[0]: seed 0, fp32, N=512 D=256 E=8 ffn_dim=1024 k=2, swiglu, aux 0.01, z-loss 1e-3."""
    gold = torch.load(os.path.join(GOLD, "layer_config1_fp32.pt"))
    N, D, E, F, k = gold["shape"]
    torch.manual_seed(gold["seed"])
    h = torch.randn(N, D)
    g = torch.randn(E, D) * 0.02
    wu = torch.randn(E, F, D) * 0.02
    wd = torch.randn(E, D, F // 2) * 0.02
    go = torch.randn(N, D)
    case = gold["cases"]["swiglu/softmax/0.01/0.001"]
    fw = orc.fused_moe_forward(h, g, wu, wd, k, "swiglu", "softmax", 0.01, 0.001, dtype=torch.float32)
    bw = orc.fused_moe_backward(fw, go)
    assert torch.equal(fw["topk_idx"].to(torch.int32), case["topk_idx"])
    assert rel(fw["out"], case["out"]) < 2e-5
    assert rel(bw["dH"], case["dH"]) < 2e-5
    assert rel(bw["dGate"], case["dGate"]) < 2e-5
    assert rel(bw["dW_up"][:, ::8, ::8], case["dW_up_s8"]) < 2e-5
    assert rel(bw["dW_down"][:, ::8, ::8], case["dW_down_s8"]) < 2e-5
    for name, v in case["losses"].items():
        assert abs(float(fw["losses"][name]) - v) <= 1e-6 * max(1.0, abs(v))


def test_oracle_backward_matches_autograd():
    """The hand-written backward equals torch autograd of a differentiable restatement (fp64)."""
    torch.manual_seed(3)
    N, D, E, F, k = 40, 32, 4, 64, 2
    h = torch.randn(N, D, dtype=torch.float64, requires_grad=True)
    g = (torch.randn(E, D, dtype=torch.float64) * 0.3).requires_grad_()
    wu = (torch.randn(E, F, D, dtype=torch.float64) * 0.2).requires_grad_()
    wd = (torch.randn(E, D, F // 2, dtype=torch.float64) * 0.2).requires_grad_()
    go = torch.randn(N, D, dtype=torch.float64)
    for gating in ("softmax", "sigmoid"):
        fw = orc.fused_moe_forward(h.detach(), g.detach(), wu.detach(), wd.detach(), k, "swiglu", gating, 0.02,
                                   0.003, dtype=torch.float64)
        bw = orc.fused_moe_backward(fw, go)
        logits = h @ g.T
        idx = fw["topk_idx"]
        if gating == "softmax":
            w = torch.softmax(logits.gather(1, idx), -1)
        else:
            sc = torch.sigmoid(logits).gather(1, idx)
            w = sc / (sc.sum(-1, keepdim=True) + orc.WEIGHT_EPS)
        out = torch.zeros(N, D, dtype=torch.float64)
        for j in range(k):
            for e in range(E):
                m = idx[:, j] == e
                if m.any():
                    x = h[m]
                    pre = x @ wu[e].T
                    a = torch.nn.functional.silu(pre[:, :F // 2]) * pre[:, F // 2:]
                    out[m] = out[m] + w[m, j:j + 1] * (a @ wd[e].T)
        ls = orc.losses(logits, w, idx, gating, 0.02, 0.003)
        loss = (out * go).sum() + ls["aux_loss"].double() + ls["z_loss"].double()
        grads = torch.autograd.grad(loss, [h, g, wu, wd])
        assert rel(fw["out"], out.detach()) < 1e-6
        for name, ref in zip(("dH", "dGate", "dW_up", "dW_down"), grads):
            assert rel(bw[name], ref) < 2e-5, (gating, name)


def test_grouped_layout_properties():
    torch.manual_seed(0)
    idx = torch.randint(0, 8, (300, 2))
    ts, pos, src = orc.grouped_layout(idx, 8)
    flat = idx.reshape(-1)
    assert (pos // 128 >= ts[flat]).all() and (pos // 128 < ts[flat + 1]).all()
    assert (src[pos] == torch.arange(flat.numel())).all()
    assert (src >= 0).sum() == flat.numel()
    # stable: inside an expert, grouped rows increase with the flat slot
    for e in range(8):
        rows = pos[flat == e]
        assert (rows[1:] > rows[:-1]).all()


def _variant_inputs(gold):
    N, D, E, F, k = gold["shape"]
    torch.manual_seed(gold["seed"])
    h = torch.randn(N, D)
    g = torch.randn(E, D) * 0.02 * gold["gate_scale"]
    wu = torch.randn(E, F, D) * 0.02
    wd = torch.randn(E, D, F // 2) * 0.02
    go = torch.randn(N, D)
    return h, g, wu, wd, go


def test_routing_variants_and_capacity_golden():
    """Group-limited / pre-softmax / biased routing and capacity dropping against the reference's slow path."""
    gold = torch.load(os.path.join(GOLD, "layer_variants_fp32.pt"))
    N, D, E, F, k = gold["shape"]
    h, g, wu, wd, go = _variant_inputs(gold)
    assert len(gold["cases"]) == 8
    for name, case in gold["cases"].items():
        extra = dict(case["extra"])
        if case["has_bias"]:
            extra["expert_bias"] = gold["bias"] * case["bias_scale"]
        fw = orc.fused_moe_forward(h, g, wu, wd, k, "swiglu", case["gating"], dtype=torch.float32, **extra)
        bw = orc.fused_moe_backward(fw, go)
        assert torch.equal(fw["topk_idx"].to(torch.int32), case["topk_idx"]), name
        assert rel(fw["out"], case["out"]) < 2e-5, name
        assert rel(bw["dH"], case["dH"]) < 2e-5 and rel(bw["dGate"], case["dGate"]) < 2e-5, name
        if "dropped" in case:
            assert int((fw["keep"] == 0).sum()) == case["dropped"] > 0, name
