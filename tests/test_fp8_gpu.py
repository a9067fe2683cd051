"""GPU: the opt-in FP8 (e4m3) forward projections of the routed experts.

Two levels. (1) The kernels against exact arithmetic on the quantised values: the GEMM accumulates products of
e4m3 numbers in fp32, so out = (q_a * s_a) (q_b * s_b)^T computed in fp32 by torch from the same quantised tensors
is the reference, and only the bf16 rounding of the output separates the two (bound 1e-2). (2) The layer with FP8
forward projections against the bf16 layer: e4m3 keeps 3 mantissa bits (relative rounding error up to 2^-4 per
element), so the stated tolerance is max |a - b| / max |b| <= 0.12 and a relative Frobenius error <= 0.08; the
routing decisions, which do not go through FP8, stay bit-identical.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

import flashfusedmoe_b200 as ffm  # noqa: E402
from flashfusedmoe_b200 import ops  # noqa: E402

DEV = "cuda"


def rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def dequant(q, scale):
    return q.view(torch.float8_e4m3fn).float() * scale[: q.shape[0]].unsqueeze(1)


def test_quantize_rows_round_trip():
    torch.manual_seed(0)
    x = (torch.randn(300, 256, device=DEV) * torch.rand(300, 1, device=DEV) * 3).bfloat16()
    x[7] = 0
    q, s = ops.quantize_rows_e4m3(x)
    amax = x.float().abs().amax(1)
    want = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    assert torch.allclose(s[:300], want, rtol=1e-6)
    back = dequant(q, s)
    assert (back[7] == 0).all()
    # e4m3 rounding: at most half a unit in the last place of a 3-bit mantissa, relative to the row's largest value
    assert ((back - x.float()).abs() <= amax.unsqueeze(1) * 2.0 ** -4 + 1e-12).all()
    ref = (x.float() / s[:300].unsqueeze(1)).to(torch.float8_e4m3fn)
    assert (q.view(torch.float8_e4m3fn).float() == ref.float()).float().mean() > 0.999


@pytest.mark.parametrize("counts,K,H", [([300, 0, 129, 64], 256, 128), ([2048] * 8, 1024, 2048)])
def test_fp8_grouped_gemms_match_exact_arithmetic_on_quantised_values(counts, K, H):
    torch.manual_seed(K + H)
    E = len(counts)
    ids = torch.cat([torch.full((c,), e, dtype=torch.int32) for e, c in enumerate(counts)]).to(DEV)
    _, ts, pos, src, rows_cap = ops.group_rows(ids, E)
    X = torch.zeros(rows_cap, K, device=DEV, dtype=torch.bfloat16)
    X[pos.long()] = torch.randn(ids.numel(), K, device=DEV).bfloat16()
    Wu = (torch.randn(E, 2 * H, K, device=DEV) * 0.05).bfloat16()
    Wd = (torch.randn(E, K, H, device=DEV) * 0.05).bfloat16()
    xq, xs = ops.quantize_rows_e4m3(X)
    wuq, wus = ops.quantize_weight_e4m3(Wu)
    act, pre = ops.grouped_gemm_glu_fp8(xq, xs, wuq, wus, E, ts, K, H, "swiglu")
    aq, as_ = ops.quantize_rows_e4m3(act)
    wdq, wds = ops.quantize_weight_e4m3(Wd)
    Y = ops.grouped_gemm_fp8(aq, as_, wdq, wds, E, ts, H, K)
    ops.check_status()
    Xd, Ad = dequant(xq, xs), dequant(aq, as_)
    Wud = wuq.view(torch.float8_e4m3fn).float() * wus.view(E, 1, 1)
    Wdd = wdq.view(torch.float8_e4m3fn).float() * wds.view(E, 1, 1)
    assert torch.allclose(wus, Wu.float().abs().amax(dim=(1, 2)) / 448.0, rtol=1e-6)
    for e in range(E):
        lo = int(ts[e]) * 128
        n = counts[e]
        if n == 0:
            continue
        p_ref = Xd[lo:lo + n] @ Wud[e].T
        assert rel(pre[lo:lo + n], p_ref) <= 1e-2, ("pre", e)
        pb = pre[lo:lo + n].float()
        a_ref = torch.nn.functional.silu(pb[:, :H]) * pb[:, H:]
        assert rel(act[lo:lo + n], a_ref) <= 1e-2, ("act", e)
        y_ref = Ad[lo:lo + n] @ Wdd[e].T
        assert rel(Y[lo:lo + n], y_ref) <= 1e-2, ("down", e)


def test_layer_with_fp8_forward_against_bf16_layer():
    torch.manual_seed(1)
    N, D, F, E, k = 4096, 1024, 4096, 8, 2
    h = torch.randn(N, D, device=DEV).bfloat16()
    g = (torch.randn(E, D, device=DEV) * 0.02).bfloat16()
    wu = (torch.randn(E, F, D, device=DEV) * 0.02).bfloat16()
    wd = (torch.randn(E, D, F // 2, device=DEV) * 0.02).bfloat16()
    go = torch.randn(N, D, device=DEV).bfloat16()

    def run():
        ps = [t.clone().requires_grad_() for t in (h, g, wu, wd)]
        out, m = ffm.fused_moe(*ps, top_k=k, return_metrics=True)
        out.backward(go)
        return out.detach(), m["tokens_per_expert"], [p.grad for p in ps]

    want, counts, grads = run()
    old = ffm.set_expert_gemm_precision("fp8")
    try:
        got, counts8, grads8 = run()
        got2, _, _ = run()
    finally:
        ffm.set_expert_gemm_precision(old)
    ops.check_status()
    assert torch.equal(counts, counts8), "routing does not go through FP8"
    assert torch.equal(got, got2), "deterministic"
    fro = ((got.float() - want.float()).norm() / want.float().norm()).item()
    print(f"[fp8 layer] out: max-norm {rel(got, want):.3e}, Frobenius {fro:.3e}; "
          + ", ".join(f"grad{i} {rel(a, b):.3e}" for i, (a, b) in enumerate(zip(grads8, grads))))
    assert rel(got, want) <= 0.12 and fro <= 0.08
    # the backward pass runs in bf16 from the saved tensors (pre-activations come from the FP8 up-projection)
    for a, b in zip(grads8, grads):
        assert torch.isfinite(a).all() and rel(a, b) <= 0.15
