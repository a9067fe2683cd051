"""GPU: gradients of every parameter through the layer at the BASELINE shapes, and the count of routing decisions
that differ from the reference's logits.

The CPU oracle cannot run these sizes, so the comparison is a plain fp32 restatement on the GPU of the reference's
hand-written backward (src/flashfusemoe/fused_moe.py:482-595), expert by expert, from the kernel's own expert
assignments. It has no bf16 rounding points; the tolerance is the bf16 bound used everywhere else (max |a - b| /
max |b| <= 2e-2). The layer call goes through the default schedule: the GLU backward rides inside the dW_down
GEMM launch and the routing backward runs on a side stream.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

import flashfusedmoe_b200 as ffm  # noqa: E402
from flashfusedmoe_b200 import _lib, ops  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

DEV = "cuda"
TOL = 2e-2
F = torch.nn.functional


def rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def zipf_bias(E, seed):
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(E, generator=g)
    p = 1.0 / torch.arange(1, E + 1).float() ** 1.1
    return torch.log(p / p.sum())[perm].to(DEV)


def fp32_layer_gradients(h, g, wu, wd, go, idx, logits, shared=None):
    """Forward and the reference's backward formulas in fp32, per expert. idx [N, k] and logits [N, E] come from the
    routing kernel (softmax over the selected logits, no bias in the weights). Returns out, dH, dGate, dW_up, dW_down
    (+ shared-expert gradients)."""
    N, D = h.shape
    E, k = g.shape[0], idx.shape[1]
    H = wu.shape[1] // 2
    hf, gf = h.float(), g.float()
    lg = logits.float()
    w = torch.softmax(lg.gather(1, idx), dim=-1)                 # [N, k] fp32
    wb = w.bfloat16().float()                                    # the combine multiplies by the bf16-rounded weight
    out = torch.zeros(N, D, device=h.device)
    dH = torch.zeros(N, D, device=h.device)
    gw = torch.zeros(N, k, device=h.device)
    dWu = torch.zeros(E, 2 * H, D, device=h.device)
    dWd = torch.zeros(E, D, H, device=h.device)
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        x = hf[tok]
        pre = x @ wu[e].float().T
        gate, up = pre[:, :H], pre[:, H:]
        s = torch.sigmoid(gate)
        a = gate * s * up
        y = a @ wd[e].float().T
        gof = go[tok].float()
        out.index_add_(0, tok, y * wb[tok, slot].unsqueeze(1))
        gw[tok, slot] = (y * gof).sum(-1)
        gy = gof * wb[tok, slot].unsqueeze(1)
        dWd[e] = gy.T @ a
        da = gy @ wd[e].float()
        gu = torch.cat([da * up * (s * (1 + gate * (1 - s))), da * gate * s], dim=1)
        dWu[e] = gu.T @ x
        dH.index_add_(0, tok, gu @ wu[e].float())
        del pre, gate, up, s, a, y, gy, da, gu
    # softmax Jacobian over the k selected logits, scattered to [N, E]
    gsel = w * (gw - (w * gw).sum(-1, keepdim=True))
    gl = torch.zeros(N, E, device=h.device).scatter_(1, idx, gsel)
    dH += gl @ gf
    dGate = gl.T @ hf
    res = dict(out=out, dH=dH, dGate=dGate, dW_up=dWu, dW_down=dWd)
    if shared is not None:
        sg, su, sd = (t.float() for t in shared)
        pg, pu = hf @ sg.T, hf @ su.T
        s = torch.sigmoid(pg)
        a = pg * s * pu
        res["out"] = out + a @ sd.T
        gof = go.float()
        res["d_shared_down"] = gof.T @ a
        da = gof @ sd
        dg, du = da * pu * (s * (1 + pg * (1 - s))), da * pg * s
        res["d_shared_gate"], res["d_shared_up"] = dg.T @ hf, du.T @ hf
        res["dH"] = dH + dg @ sg + du @ su
    return res


def layer_case(N, D, Fdim, E, k, seed, bias=None, shared_ffn=None):
    torch.manual_seed(seed)
    H = Fdim // 2
    h = torch.randn(N, D, device=DEV).bfloat16().requires_grad_()
    g = (torch.randn(E, D, device=DEV) * 0.02).bfloat16().requires_grad_()
    wu = (torch.randn(E, Fdim, D, device=DEV) * 0.02).bfloat16().requires_grad_()
    wd = (torch.randn(E, D, H, device=DEV) * 0.02).bfloat16().requires_grad_()
    go = torch.randn(N, D, device=DEV).bfloat16()
    shared = None
    addend = None
    if shared_ffn is not None:
        Hs = shared_ffn // 2
        shared = [(torch.randn(Hs, D, device=DEV) * 0.02).bfloat16().requires_grad_() for _ in range(2)]
        shared.append((torch.randn(D, Hs, device=DEV) * 0.02).bfloat16().requires_grad_())
        from flashfusedmoe_b200.fused_moe import glu_ffn
        addend = glu_ffn(h, *shared)
    out, losses = ffm.fused_moe(h, g, wu, wd, top_k=k, expert_bias=bias, return_metrics=True, _addend=addend)
    out.backward(go)
    ops.check_status()
    r = ops.route_forward(h.detach(), g.detach(), k, "softmax", bias)
    ref = fp32_layer_gradients(h.detach(), g.detach(), wu.detach(), wd.detach(), go, r.topk_idx.long(), r.logits,
                               None if shared is None else [t.detach() for t in shared])
    errs = {"out": rel(out, ref["out"]), "dH": rel(h.grad, ref["dH"]), "dGate": rel(g.grad, ref["dGate"]),
            "dW_up": rel(wu.grad, ref["dW_up"]), "dW_down": rel(wd.grad, ref["dW_down"])}
    if shared is not None:
        errs.update(d_shared_gate=rel(shared[0].grad, ref["d_shared_gate"]),
                    d_shared_up=rel(shared[1].grad, ref["d_shared_up"]),
                    d_shared_down=rel(shared[2].grad, ref["d_shared_down"]))
    print(f"[gradient parity] N={N} D={D} F={Fdim} E={E} k={k}:", {n: f"{v:.2e}" for n, v in errs.items()})
    bad = {n: v for n, v in errs.items() if not v <= TOL}
    assert not bad, bad
    # a strided sample (every 8th row and column), compared element-wise against its own scale: a whole block of a
    # weight gradient that is wrong but small would hide in the maximum norm of the full tensor
    for name, ours in (("dW_up", wu.grad), ("dW_down", wd.grad)):
        for e in range(E):
            a, b = ours[e, ::8, ::8].float(), ref[name][e, ::8, ::8]
            if b.abs().max() > 0:
                assert rel(a, b) <= TOL, (name, e, rel(a, b))


def test_config2_layer_gradients_full_shape():
    """BASELINE configs[1]: 16,384 tokens, D 1024, ffn_dim 4096, 8 experts, top-2, one shared expert (ffn_dim 4096)."""
    layer_case(16384, 1024, 4096, 8, 2, seed=1, shared_ffn=4096)


def test_config3_layer_gradients_full_shape():
    """BASELINE configs[2]: 8,192 tokens, D 4096, ffn_dim 2 x 14336, 8 experts, top-2, Zipf(1.1) gate bias."""
    layer_case(8192, 4096, 28672, 8, 2, seed=2, bias=zipf_bias(8, 2))


def test_config4_layer_gradients_full_shape():
    """BASELINE configs[3] local shape: 16,384 tokens, D 2048, ffn_dim 2 x 1408, 64 experts, top-6."""
    layer_case(16384, 2048, 2816, 64, 6, seed=3)


def test_split_weight_gradient_path():
    """The weight-gradient GEMM of a rank with few local experts is cut along the token dimension so that its output
    tiles fill the GPU (fused_moe._grouped_wgrad); one and two local experts at the benchmark's expert-parallel shapes,
    with and without the GLU backward riding along, against fp32."""
    import sys
    fm = sys.modules["flashfusedmoe_b200.fused_moe"]
    torch.manual_seed(11)
    for groups, rows_per, M, Nn in ((1, 32768, 1024, 2048), (2, 16384, 512, 2048), (1, 8192, 2048, 1024)):
        counts = [rows_per - 37 * (i + 1) for i in range(groups)]
        ids = torch.cat([torch.full((c,), i, dtype=torch.int32) for i, c in enumerate(counts)]).to(DEV)
        _, ts, pos, src, rows_cap = ops.group_rows(ids, groups)
        A = torch.zeros(rows_cap, M, device=DEV, dtype=torch.bfloat16)
        B = torch.zeros(rows_cap, Nn, device=DEV, dtype=torch.bfloat16)
        A[pos.long()] = torch.randn(ids.numel(), M, device=DEV).bfloat16()
        B[pos.long()] = torch.randn(ids.numel(), Nn, device=DEV).bfloat16()
        assert fm._wgrad_split_factor(groups, M, Nn) > 1, "this shape is meant to take the split path"
        got = fm._grouped_wgrad(A, B, groups, ts, scale=0.5)
        d_act = torch.randn(rows_cap, Nn, device=DEV).bfloat16()
        pre = torch.randn(rows_cap, 2 * Nn, device=DEV).bfloat16()
        got_p, gU = fm._grouped_wgrad(A, B, groups, ts, scale=0.5, passenger=(d_act, pre, "swiglu"))
        ops.check_status()
        assert torch.equal(got, got_p), "the passenger must not change the GEMM's result"
        assert torch.equal(gU[: int(ts[-1]) * 128], ops.glu_backward(d_act, pre, ts, groups, "swiglu")[: int(ts[-1]) * 128])
        for e in range(groups):
            lo = int(ts[e]) * 128
            want = 0.5 * (A[lo:lo + counts[e]].float().T @ B[lo:lo + counts[e]].float())
            assert rel(got[e], want) <= 1e-2, (groups, e, rel(got[e], want))


# ---- routing decisions against the reference's logits ----------------------------------------------------------

CONFIG_ROUTING = [
    # name, tokens, D, E, k, seed, Zipf bias, share of tokens allowed to differ
    ("configs[1]", 16384, 1024, 8, 2, 1, False, 2e-4),
    ("configs[2]", 8192, 4096, 8, 2, 2, True, 2e-4),
    ("configs[3]", 16384, 2048, 64, 6, 3, False, 2e-3),
    ("configs[4]", 128, 7168, 256, 8, 4, False, 2e-2),
]


def bf16_ulps_apart(a, b):
    ai = a.view(torch.int16).to(torch.int32)
    bi = b.view(torch.int16).to(torch.int32)
    ai = torch.where(ai < 0, -(ai & 0x7FFF), ai)
    bi = torch.where(bi < 0, -(bi & 0x7FFF), bi)
    return (ai - bi).abs()


@pytest.mark.parametrize("name,N,D,E,k,seed,biased,allowed", CONFIG_ROUTING)
def test_assignments_against_reference_logits(name, N, D, E, k, seed, biased, allowed):
    """The reference routes on the bf16 output of a cuBLAS GEMM with fp32 accumulation (fused_moe.py:334,
    kernels/fused_topk.py:53-70). Here: the same logits from an fp32 matmul rounded to bf16, the reference rule on
    them (oracle), and the count of tokens whose expert set differs from the fused kernel's. Every such token must owe
    it to logits that the two GEMMs round differently (accumulation order), by one bf16 unit in the last place for
    the CUDA-core gate GEMM (E <= 32); the tensor-core gate GEMM (E > 32) truncates its fp32 additions, so there the
    bound is the accumulation error itself. Target 0; the allowed share is the ceiling before it needs a look."""
    torch.manual_seed(seed)
    h = torch.randn(N, D, device=DEV).bfloat16()
    g = (torch.randn(E, D, device=DEV) * 0.02).bfloat16()
    bias = zipf_bias(E, seed) if biased else None
    r = ops.route_forward(h, g, k, "softmax", bias)
    ops.check_status()
    ref32 = h.float() @ g.float().T
    ref_logits = ref32.bfloat16()
    _, i_ref = orc.route(ref_logits.cpu(), "softmax", k, None if bias is None else bias.cpu())
    i_ref = i_ref.to(DEV)
    differs = (r.topk_idx.long().sort(1).values != i_ref.sort(1).values).any(1)
    count = int(differs.sum())
    order_differs = int((r.topk_idx.long() != i_ref).any(1).sum()) - count
    logit_rows_differ = int((r.logits != ref_logits).any(1).sum())
    print(f"[routing vs reference logits] {name}: {count} of {N} tokens with a different expert set "
          f"({order_differs} more with the same set in another order; {logit_rows_differ} rows with any logit "
          f"rounded differently)")
    if count:
        rows = differs.nonzero().squeeze(1)
        apart = bf16_ulps_apart(r.logits[rows], ref_logits[rows])
        assert (apart.max(1).values >= 1).all(), "a differing assignment without a differing logit"
        if E <= 32:
            assert (apart <= 1).all(), "logit difference of more than one bf16 unit in the last place"
        else:
            acc_err = 1.5e-5 * (h[rows].float().abs() @ g.float().abs().T)
            ulp = torch.maximum(r.logits[rows].float().abs(), ref_logits[rows].float().abs()) * 2.0 ** -7
            assert ((r.logits[rows].float() - ref_logits[rows].float()).abs() <= ulp + acc_err).all()
    assert count <= max(1, int(allowed * N)), f"{count} of {N} tokens routed differently"
    # rows whose logits agree are routed identically, order included
    same_rows = (r.logits == ref_logits).all(1)
    assert torch.equal(r.topk_idx.long()[same_rows], i_ref[same_rows])


# ---- robustness ------------------------------------------------------------------------------------------------

def test_capacity_dropping_without_gradients_is_finite_and_equal():
    """With capacity_factor a dropped slot keeps weight 0 and a grouped row nobody fills. Under no_grad the padding
    rows are otherwise left uninitialised, and 0 * NaN would reach the output: fill the allocator's free blocks with
    bf16 NaNs first, then compare the no_grad output with the grad-enabled one."""
    torch.manual_seed(5)
    N, D, Fdim, E, k = 1024, 256, 512, 8, 2
    h = torch.randn(N, D, device=DEV).bfloat16()
    g = (torch.randn(E, D, device=DEV) * 0.3).bfloat16()      # skewed routing: some experts overflow their capacity
    wu = (torch.randn(E, Fdim, D, device=DEV) * 0.05).bfloat16()
    wd = (torch.randn(E, D, Fdim // 2, device=DEV) * 0.05).bfloat16()
    hg = h.clone().requires_grad_()
    want, m = ffm.fused_moe(hg, g, wu, wd, top_k=k, capacity_factor=0.5, return_metrics=True)
    assert int(m["dropped_token_count"]) > 0, "the case must drop rows"
    rows_cap = ops.rows_capacity(N * k, E)
    for shape in ((rows_cap, D), (rows_cap, Fdim // 2), (rows_cap, Fdim), (N, D)):
        junk = [torch.full(shape, float("nan"), device=DEV, dtype=torch.bfloat16) for _ in range(3)]
        del junk
    with torch.no_grad():
        got, _ = ffm.fused_moe(h, g, wu, wd, top_k=k, capacity_factor=0.5)
    ops.check_status()
    assert torch.isfinite(got).all()
    assert torch.equal(got, want.detach())


def test_peer_wait_runs_out_and_the_failure_surfaces():
    """A bounded device wait that runs out: the flag barrier of a two-rank exchange on ONE GPU, both flag arrays
    local, the peer's slot never written, a budget of 1e5 cycles. The kernel returns by itself with status 105
    (nothing hangs, the GPU stays usable), check_status raises, and so does a later fused_moe() call through the
    asynchronous poll of the status word."""
    import ctypes
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    ops.check_status()
    flags = torch.zeros(2, 64, dtype=torch.int32, device=DEV)
    arrays = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    st = ops.status_tensor(dev)

    def expire():
        rc = lib.ffm_p2p_signal_wait(arrays, 0, 2, 1, st.data_ptr(), 100000, ops._stream())
        assert rc == 0
        torch.cuda.synchronize()

    expire()
    assert int(flags[1, 0]) == 1 and int(flags[0, 0]) == 1, "rank 0 published its epoch to both flag arrays"
    assert int(flags[0, 1]) == 0, "nobody plays rank 1"
    with pytest.raises(RuntimeError, match="105"):
        ops.check_status()
    assert int(st.item()) == 0, "check_status clears the word"
    # the GPU is usable straight away
    x = torch.randn(256, 256, device=DEV)
    assert torch.isfinite(x @ x).all()

    # the same failure seen by the product path: fused_moe() polls the word without waiting for the GPU
    torch.manual_seed(0)
    N, D, Fdim, E, k = 64, 64, 128, 4, 2
    h = torch.randn(N, D, device=DEV).bfloat16()
    g = torch.randn(E, D, device=DEV).bfloat16()
    wu = (torch.randn(E, Fdim, D, device=DEV) * 0.05).bfloat16()
    wd = (torch.randn(E, D, Fdim // 2, device=DEV) * 0.05).bfloat16()
    ffm.fused_moe(h, g, wu, wd, top_k=k)
    torch.cuda.synchronize()
    ffm.fused_moe(h, g, wu, wd, top_k=k)      # reads a clean word, queues the next copy
    torch.cuda.synchronize()
    expire()
    with pytest.raises(RuntimeError, match="105"):
        for _ in range(3):                    # the first call queues the copy that carries the code, a later one reads it
            ffm.fused_moe(h, g, wu, wd, top_k=k)
            torch.cuda.synchronize()
    ops.check_status()
    out, _ = ffm.fused_moe(h, g, wu, wd, top_k=k)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
