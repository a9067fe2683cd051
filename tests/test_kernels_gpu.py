"""Kernel-level checks of libffmoe on a B200: every C-ABI entry point against a plain torch fp32
restatement of the same operation, at small ragged shapes and at the single-GPU benchmark shape."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from flashfusedmoe_b200 import _lib, ops  # noqa: E402

DEV = "cuda"


def bf16_ulp_close(a, b, ulps=1):
    """True where two bf16 tensors differ by at most `ulps` units in the last place."""
    ai = a.view(torch.int16).to(torch.int32)
    bi = b.view(torch.int16).to(torch.int32)
    # map sign-magnitude to a monotonic integer line
    ai = torch.where(ai < 0, -(ai & 0x7FFF), ai)
    bi = torch.where(bi < 0, -(bi & 0x7FFF), bi)
    return (ai - bi).abs() <= ulps


def rel_err(a, b):
    a = a.float()
    b = b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def triton_rule_topk(sel, k):
    """Iterative argmax, lowest index wins ties, descending order (kernels/fused_topk.py:53-70)."""
    N, E = sel.shape
    sel = sel.clone()
    ar = torch.arange(E, device=sel.device).expand(N, E)
    out = []
    for _ in range(k):
        m = sel.max(dim=1, keepdim=True).values
        idx = torch.where(sel == m, ar, torch.full_like(ar, E)).min(dim=1).values
        out.append(idx)
        sel[torch.arange(N, device=sel.device), idx] = float("-inf")
    return torch.stack(out, dim=1)


def make_groups(counts, device=DEV):
    """tile_start / src / pos for given per-expert row counts (stable order = arrival order)."""
    E = len(counts)
    ids = torch.cat([torch.full((c,), e, dtype=torch.int32) for e, c in enumerate(counts)])
    ids = ids[torch.randperm(ids.numel())].contiguous().to(device)
    return ids


@pytest.mark.parametrize("gating", ["softmax", "sigmoid"])
@pytest.mark.parametrize("N,D,E,k", [(1, 64, 4, 1), (37, 64, 8, 2), (512, 256, 8, 2), (300, 128, 16, 4),
                                     (129, 256, 64, 6), (128, 512, 256, 8), (1000, 128, 24, 3), (700, 256, 32, 4)])
def test_route_forward(N, D, E, k, gating):
    torch.manual_seed(N + E)
    hidden = torch.randn(N, D, device=DEV).bfloat16()
    gate = (torch.randn(E, D, device=DEV) * 0.5).bfloat16()
    r = ops.route_forward(hidden, gate, k, gating)
    ops.check_status()
    ref32 = hidden.float() @ gate.float().T
    ref_logits = ref32.bfloat16()
    # one bf16 unit in the last place, or (for logits that cancel to nearly zero) the fp32 accumulation-order error
    acc_err = 4e-6 * (hidden.float().abs() @ gate.float().abs().T)
    close = bf16_ulp_close(r.logits, ref_logits, 1) | ((r.logits.float() - ref32).abs() <= acc_err + ref32.abs() * 2.0 ** -8)
    assert close.all(), "gate GEMM logits differ by more than 1 bf16 ulp"
    lg = r.logits.float()
    sel = torch.sigmoid(lg) if gating == "sigmoid" else lg
    idx_ref = triton_rule_topk(sel, k)
    if gating == "softmax":
        assert torch.equal(r.topk_idx.long(), idx_ref), "expert assignment differs from the lowest-index rule"
        w_ref = torch.softmax(lg.gather(1, idx_ref), dim=-1)
    else:
        # The kernel scores with 1 / (1 + exp(-x)), every step correctly rounded in fp32. torch's CUDA sigmoid can
        # differ from that by a unit in the last place, which changes the choice only where scores (nearly) tie:
        # saturated scores close to 1 above all (these logits reach |x| > 20). So: the k experts are distinct, each
        # of them scores at least the reference's k-th best score minus 2 fp32 ulp (a legitimate top-k up to such
        # ties), and almost every row picks exactly the reference's set.
        ours = r.topk_idx.long()
        assert (ours.sort(1).values.diff(dim=1) > 0).all(), "an expert was selected twice"
        sig = torch.sigmoid(lg)
        kth = sig.gather(1, idx_ref)[:, -1:]
        assert (sig.gather(1, ours) >= kth - 2.0 * kth * 2.0 ** -23).all(), "a selected expert is not a top-k tie"
        same = (ours.sort(1).values == idx_ref.sort(1).values).all(1)
        assert same.float().mean() > 0.99
        sc = sig.gather(1, ours)
        w_ref = sc / (sc.sum(-1, keepdim=True) + 1e-6)
    assert torch.allclose(r.topk_w, w_ref, atol=2e-6, rtol=1e-4)
    assert torch.allclose(r.lse, torch.logsumexp(lg, dim=-1), atol=1e-4, rtol=1e-5)
    flat = r.topk_idx.long().view(-1)
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(r.counts.long(), counts)
    tiles = 2 * ((counts + 255) // 256)
    ts = torch.zeros(E + 1, dtype=torch.long, device=DEV)
    ts[1:] = torch.cumsum(tiles, 0)
    assert torch.equal(r.tile_start.long(), ts)
    # stable grouped order: within an expert rows follow flat slot order
    order = torch.argsort(flat, stable=True)
    starts = torch.zeros(E + 1, dtype=torch.long, device=DEV)
    starts[1:] = torch.cumsum(counts, 0)
    rank = torch.arange(flat.numel(), device=DEV) - starts[flat[order]]
    pos_ref = torch.empty_like(flat)
    pos_ref[order] = ts[flat[order]] * 128 + rank
    assert torch.equal(r.pos.long(), pos_ref)
    src_ref = torch.full((r.rows_cap,), -1, dtype=torch.long, device=DEV)
    src_ref[pos_ref] = torch.arange(flat.numel(), device=DEV)
    assert torch.equal(r.src.long()[: r.rows_cap], src_ref)
    # loss statistics
    if gating == "softmax":
        mass = torch.zeros(E, device=DEV).scatter_add_(0, flat, r.topk_w.view(-1))
    else:
        mass = torch.sigmoid(lg).sum(0)
    assert torch.allclose(r.stats[:E], mass, rtol=1e-4, atol=1e-4)
    assert torch.allclose(r.stats[E], (r.lse ** 2).sum(), rtol=1e-4)
    assert torch.allclose(r.stats[E + 1], (counts.float() * mass).sum(), rtol=1e-4)


def test_route_forward_bias_and_scale():
    torch.manual_seed(3)
    N, D, E, k = 256, 128, 8, 2
    hidden = torch.randn(N, D, device=DEV).bfloat16()
    gate = (torch.randn(E, D, device=DEV) * 0.1).bfloat16()
    bias = torch.randn(E, device=DEV)
    r = ops.route_forward(hidden, gate, k, "softmax", expert_bias=bias, weight_scale=2.5 / k)
    lg = r.logits.float()
    idx_ref = triton_rule_topk(lg + bias, k)
    assert torch.equal(r.topk_idx.long(), idx_ref)
    w_ref = torch.softmax(lg.gather(1, idx_ref), -1) * (2.5 / k)
    assert torch.allclose(r.topk_w, w_ref, atol=2e-6, rtol=1e-4)


def test_group_rows_and_permute():
    torch.manual_seed(5)
    counts = [0, 130, 1, 255, 0, 64, 128, 7]
    ids = make_groups(counts)
    T, E = ids.numel(), len(counts)
    c, ts, pos, src, rows_cap = ops.group_rows(ids, E)
    ops.check_status()
    assert c.tolist() == counts
    assert ts.tolist() == [0] + torch.cumsum(2 * ((torch.tensor(counts) + 255) // 256), 0).tolist()
    order = torch.argsort(ids.long(), stable=True)
    starts = torch.zeros(E + 1, dtype=torch.long, device=DEV)
    starts[1:] = torch.cumsum(torch.tensor(counts, device=DEV), 0)
    rank = torch.arange(T, device=DEV) - starts[ids.long()[order]]
    pos_ref = torch.empty(T, dtype=torch.long, device=DEV)
    pos_ref[order] = ts.long()[ids.long()[order]] * 128 + rank
    assert torch.equal(pos.long(), pos_ref)
    x = torch.randn(T, 64, device=DEV).bfloat16()
    g = ops.permute_rows(x, src, rows_cap, 1)
    ref = torch.zeros(rows_cap, 64, device=DEV, dtype=torch.bfloat16)
    ref[pos_ref] = x
    assert torch.equal(g, ref)


def _grouped_case(counts, K, dev=DEV):
    ids = make_groups(counts)
    E = len(counts)
    c, ts, pos, src, rows_cap = ops.group_rows(ids, E)
    x = torch.randn(ids.numel(), K, device=dev).bfloat16()
    A = ops.permute_rows(x, src, rows_cap, 1)
    row_expert = torch.full((rows_cap,), -1, dtype=torch.long, device=dev)
    row_expert[pos.long()] = ids.long()
    return A, ts, row_expert, rows_cap


GEMM_SHAPES = [([5, 0, 200, 128], 64, 64), ([300, 17, 129, 64, 1, 0, 77, 256], 128, 320),
               ([100] * 3, 256, 96), ([2048] * 8, 1024, 1024)]


@pytest.mark.parametrize("counts,K,Nout", GEMM_SHAPES)
def test_grouped_gemm_kmajor(counts, K, Nout):
    torch.manual_seed(K + Nout)
    A, ts, row_expert, rows_cap = _grouped_case(counts, K)
    E = len(counts)
    B = (torch.randn(E, Nout, K, device=DEV) * 0.05).bfloat16()
    out = ops.grouped_gemm(A, B, _lib.B_KMAJOR, E, ts, K, Nout)
    ops.check_status()
    used = int(ts[-1].item()) * 128
    for e in range(E):
        rows = (row_expert == e).nonzero().view(-1)
        if rows.numel() == 0:
            continue
        ref = A[rows].float() @ B[e].float().T
        assert rel_err(out[rows], ref) < 1e-2, f"expert {e}"
    pad = (row_expert[:used] == -1).nonzero().view(-1)
    assert (out[pad] == 0).all()


@pytest.mark.parametrize("counts,K,Nout", GEMM_SHAPES)
def test_grouped_gemm_nmajor(counts, K, Nout):
    if Nout % 64:
        pytest.skip("N-major B needs Nout % 64 == 0")
    torch.manual_seed(K + Nout + 1)
    A, ts, row_expert, rows_cap = _grouped_case(counts, K)
    E = len(counts)
    B = (torch.randn(E, K, Nout, device=DEV) * 0.05).bfloat16()
    out = ops.grouped_gemm(A, B, _lib.B_NMAJOR, E, ts, K, Nout, scale=0.5)
    ops.check_status()
    for e in range(E):
        rows = (row_expert == e).nonzero().view(-1)
        if rows.numel() == 0:
            continue
        ref = 0.5 * (A[rows].float() @ B[e].float())
        assert rel_err(out[rows], ref) < 1e-2, f"expert {e}"


@pytest.mark.parametrize("rows,K,Nout", [(1, 64, 32), (130, 128, 288), (4096, 1024, 512)])
def test_dense_gemm(rows, K, Nout):
    torch.manual_seed(rows)
    A = torch.randn(rows, K, device=DEV).bfloat16()
    B = (torch.randn(Nout, K, device=DEV) * 0.05).bfloat16()
    out = ops.grouped_gemm(A, B, _lib.B_KMAJOR, 1, None, K, Nout)
    ops.check_status()
    assert rel_err(out, A.float() @ B.float().T) < 1e-2
    if Nout % 64 == 0:
        Bt = B.T.contiguous()
        out2 = ops.grouped_gemm(A, Bt, _lib.B_NMAJOR, 1, None, K, Nout)
        ops.check_status()
        assert rel_err(out2, A.float() @ B.float().T) < 1e-2


def glu_ref(act, g, u):
    if act == "swiglu":
        return torch.nn.functional.silu(g) * u
    if act == "geglu":
        return torch.nn.functional.gelu(g, approximate="tanh") * u
    if act == "geglu_erf":
        return torch.nn.functional.gelu(g) * u
    return torch.relu(g).square() * u


@pytest.mark.parametrize("activation", ["swiglu", "geglu", "relu_squared", "geglu_erf"])
@pytest.mark.parametrize("counts,K,H", [([5, 0, 200, 128], 64, 64), ([300, 17, 129, 64], 128, 192),
                                        ([2048] * 8, 1024, 2048)])
def test_grouped_gemm_glu(counts, K, H, activation):
    if activation != "swiglu" and H > 1000:
        pytest.skip("large shape once")
    torch.manual_seed(H)
    A, ts, row_expert, rows_cap = _grouped_case(counts, K)
    E = len(counts)
    W = (torch.randn(E, 2 * H, K, device=DEV) * 0.05).bfloat16()
    act, pre = ops.grouped_gemm_glu(A, W, W.view(-1, K)[H:], 2 * H, E, ts, K, H, activation)
    ops.check_status()
    for e in range(E):
        rows = (row_expert == e).nonzero().view(-1)
        if rows.numel() == 0:
            continue
        full = (A[rows].float() @ W[e].float().T).bfloat16()
        assert rel_err(pre[rows], full) < 1e-2, f"preact expert {e}"
        g, u = pre[rows][:, :H].float(), pre[rows][:, H:].float()
        assert rel_err(act[rows], glu_ref(activation, g, u)) < 1e-2, f"act expert {e}"


@pytest.mark.parametrize("counts,M,Nout", [([5, 0, 200, 128], 64, 64), ([300, 17, 129, 64], 192, 320),
                                           ([2048] * 8, 1024, 2048)])
def test_grouped_gemm_wgrad(counts, M, Nout):
    torch.manual_seed(M)
    A, ts, row_expert, rows_cap = _grouped_case(counts, M)
    E = len(counts)
    Bx = torch.randn(rows_cap, Nout, device=DEV).bfloat16()
    Bx[row_expert == -1] = 0
    dW = ops.grouped_gemm_wgrad(A, Bx, E, ts, scale=0.25)
    ops.check_status()
    for e in range(E):
        rows = (row_expert == e).nonzero().view(-1)
        ref = 0.25 * (A[rows].float().T @ Bx[rows].float())
        if rows.numel() == 0:
            assert (dW[e] == 0).all()
        else:
            assert rel_err(dW[e], ref) < 1e-2, f"expert {e}"


@pytest.mark.parametrize("N,D,E,k", [(7, 64, 4, 1), (300, 128, 8, 2), (128, 72, 16, 5), (16384, 1024, 8, 2)])
def test_combine_forward_backward(N, D, E, k):
    torch.manual_seed(N)
    hidden = torch.randn(N, D, device=DEV).bfloat16()
    gate = (torch.randn(E, D, device=DEV) * 0.3).bfloat16()
    r = ops.route_forward(hidden, gate, k, "softmax")
    Y = torch.randn(r.rows_cap, D, device=DEV).bfloat16()
    add = torch.randn(N, D, device=DEV).bfloat16()
    pos = r.pos.long().view(N, k)
    wb = r.topk_w.bfloat16().float()
    ref = (Y[pos].float() * wb.unsqueeze(-1)).sum(1)
    out = ops.combine_forward(Y, r.pos, r.topk_w, N, k)
    assert rel_err(out, ref) < 1e-2
    out2 = ops.combine_forward(Y, r.pos, r.topk_w, N, k, addend=add)
    assert rel_err(out2, ref.bfloat16().float() + add.float()) < 1e-2
    out3 = ops.combine_forward(Y, r.pos, None, N, k)
    assert rel_err(out3, Y[pos].float().sum(1)) < 1e-2
    go = torch.randn(N, D, device=DEV).bfloat16()
    gYw, gw = ops.combine_backward(go, Y, r.topk_w, r.src, r.rows_cap, k)
    gw_ref = (Y[pos].float() * go.float().unsqueeze(1)).sum(-1)
    assert torch.allclose(gw.view(N, k), gw_ref, rtol=1e-3, atol=1e-2)
    gYw_ref = torch.zeros(r.rows_cap, D, device=DEV)
    gYw_ref[pos.view(-1)] = (go.float().unsqueeze(1) * wb.unsqueeze(-1)).reshape(N * k, D)
    assert rel_err(gYw, gYw_ref) < 1e-2
    assert (gYw[r.src.long()[: r.rows_cap] < 0] == 0).all()


@pytest.mark.parametrize("activation", ["swiglu", "geglu", "relu_squared", "geglu_erf"])
def test_glu_backward(activation):
    torch.manual_seed(11)
    rows, H = 257, 72
    pre = torch.randn(rows, 2 * H, device=DEV).bfloat16()
    dA = torch.randn(rows, H, device=DEV).bfloat16()
    gU = ops.glu_backward(dA, pre, None, 1, activation)
    p = pre.float().requires_grad_()
    glu_ref(activation, p[:, :H], p[:, H:]).backward(dA.float())
    assert rel_err(gU, p.grad) < 2e-2


@pytest.mark.parametrize("gating", ["softmax", "sigmoid"])
@pytest.mark.parametrize("N,D,E,k", [(33, 64, 4, 2), (512, 256, 8, 2), (200, 128, 64, 6), (64, 2048, 256, 8),
                                     (2500, 256, 64, 6), (1024, 128, 128, 4)])  # the last two: dGate on tensor cores
def test_route_backward(N, D, E, k, gating):
    torch.manual_seed(N + k)
    hidden = torch.randn(N, D, device=DEV).bfloat16()
    gate = (torch.randn(E, D, device=DEV) * 0.3).bfloat16()
    r = ops.route_forward(hidden, gate, k, gating)
    gw = torch.randn(N, k, device=DEV)
    gaux = torch.randn(E, device=DEV)
    gz = 0.37
    dH0 = torch.randn(N, D, device=DEV).bfloat16()
    dH, dGate = ops.route_backward(gw.view(-1), r, gaux, torch.tensor(gz, device=DEV), hidden, gate, gating,
                                   dH=dH0.clone())
    # torch restatement from the kernel's own logits / indices
    lg = r.logits.float().requires_grad_()
    idx = r.topk_idx.long()
    if gating == "softmax":
        w = torch.softmax(lg.gather(1, idx), -1)
        P = torch.zeros(E, device=DEV).scatter_add(0, idx.view(-1), w.view(-1)) / N
    else:
        sc = torch.sigmoid(lg)
        ts_ = sc.gather(1, idx)
        w = ts_ / (ts_.sum(-1, keepdim=True) + 1e-6)
        P = sc.mean(0)
    loss = (w * gw).sum() + (P * gaux).sum() + gz * torch.logsumexp(lg, -1).square().mean()
    loss.backward()
    gl = lg.grad.bfloat16().float()
    dH_ref = dH0.float() + (gl @ gate.float()).bfloat16().float()
    dG_ref = gl.T @ hidden.float()
    assert rel_err(dH, dH_ref) < 2e-2
    assert rel_err(dGate, dG_ref) < 2e-2


@pytest.mark.parametrize("tile_rows", [128, 256])
def test_grouped_gemm_skips_tiles_without_valid_rows(tile_rows):
    """valid_rows / tile_rows: rows of tiles that hold valid rows are bit-identical to the full computation; tiles
    beyond a group's valid rows are left unwritten."""
    torch.manual_seed(17)
    counts = [5, 0, 200, 128, 300, 1, 129]
    K, H = 128, 192
    A, ts, row_expert, rows_cap = _grouped_case(counts, K)
    E = len(counts)
    cnt = torch.tensor(counts, dtype=torch.int32, device=DEV)
    W = (torch.randn(E, 2 * H, K, device=DEV) * 0.05).bfloat16()
    Wd = (torch.randn(E, K, H, device=DEV) * 0.05).bfloat16()
    act_full, _ = ops.grouped_gemm_glu(A, W, W.view(-1, K)[H:], 2 * H, E, ts, K, H, "swiglu", want_preact=False)
    y_full = ops.grouped_gemm(act_full, Wd, _lib.B_KMAJOR, E, ts, H, K)
    act, _ = ops.grouped_gemm_glu(A, W, W.view(-1, K)[H:], 2 * H, E, ts, K, H, "swiglu", want_preact=False,
                                  valid_rows=cnt, tile_rows=tile_rows)
    sentinel = torch.full_like(y_full, 7.0)
    lib = _lib.load()
    rc = lib.ffm_grouped_gemm(act.data_ptr(), Wd.data_ptr(), _lib.B_KMAJOR, E, ts.data_ptr(), rows_cap, H, K, 1.0,
                              sentinel.data_ptr(), cnt.data_ptr(), tile_rows, ops.status_tensor(A.device).data_ptr(),
                              torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    ops.check_status()
    valid = row_expert >= 0
    assert torch.equal(act[valid], act_full[valid])
    assert torch.equal(sentinel[valid], y_full[valid])
    # rows of tiles (128 rows, or 256 for the pair shape) that start beyond a group's valid rows were not touched
    tsl = ts.tolist()
    for e, c in enumerate(counts):
        first_untouched = tsl[e] * 128 + (c + tile_rows - 1) // tile_rows * tile_rows
        end = tsl[e + 1] * 128
        if first_untouched < end:
            assert (sentinel[first_untouched:end] == 7.0).all(), e


def test_compact_positions_matches_stable_sort():
    torch.manual_seed(23)
    N, D, E, k = 700, 64, 16, 3
    hidden = torch.randn(N, D, device=DEV).bfloat16()
    gate = (torch.randn(E, D, device=DEV) * 0.3).bfloat16()
    r = ops.route_forward(hidden, gate, k, "softmax")
    cpos, src_c = ops.compact_positions(r, N * k)
    ops.check_status()
    order = torch.argsort(r.topk_idx.view(-1).long(), stable=True)        # flat slots sorted by expert
    assert torch.equal(src_c.long(), order)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(N * k, device=DEV)
    assert torch.equal(cpos.long(), inv)


@pytest.mark.parametrize("ep,e_local", [(2, 4), (4, 2), (8, 1), (8, 32), (16, 16)])
def test_device_exchange_plan_matches_host_plan(ep, e_local):
    """ffm_p2p_plan (device) against p2p.SegmentPlan (host): same runs, ends, padding, tile_start and totals."""
    import numpy as np
    from flashfusedmoe_b200.p2p import SegmentPlan
    rng = np.random.default_rng(ep * 100 + e_local)
    E = ep * e_local
    C = rng.integers(0, 600, size=(ep, E))
    C[rng.random((ep, E)) < 0.25] = 0
    C[:, E // 2] = 0
    lib = _lib.load()
    Cd = torch.tensor(C, dtype=torch.int32, device=DEV)
    i64 = dict(dtype=torch.int64, device=DEV)
    for rank in (0, ep - 1, ep // 2):
        host = SegmentPlan(C, e_local, rank)
        d, de = torch.empty(E, 4, **i64), torch.empty(E, **i64)
        c, ce = torch.empty(e_local * ep, 4, **i64), torch.empty(e_local * ep, **i64)
        p, pe = torch.empty(e_local, 4, **i64), torch.empty(e_local, **i64)
        ts = torch.empty(e_local + 1, dtype=torch.int32, device=DEV)
        tot = torch.empty(4, **i64)
        st = ops.status_tensor(torch.device("cuda", torch.cuda.current_device()))
        stream = torch.cuda.current_stream().cuda_stream
        largest = int(host.rows_grouped.max())

        def plan(bound):
            return lib.ffm_p2p_plan(Cd.data_ptr(), ep, e_local, rank, d.data_ptr(), de.data_ptr(), c.data_ptr(),
                                    ce.data_ptr(), p.data_ptr(), pe.data_ptr(), ts.data_ptr(), tot.data_ptr(), bound,
                                    st.data_ptr(), stream)

        # a bound below the largest grouped layout of ANY rank: tables that move nothing, status 106
        assert plan(largest - 256) == 0
        torch.cuda.synchronize()
        assert int(d[:, 2].sum()) == 0 and int(c[:, 2].sum()) == 0 and int(p[:, 2].sum()) == 0
        assert tot.cpu().tolist() == [0, 0, 0, 0] and ts.cpu().tolist() == [0] * (e_local + 1)
        with pytest.raises(RuntimeError, match="106"):
            ops.check_status()
        # a bound that fits (and no bound): the full plan
        assert plan(largest) == 0
        torch.cuda.synchronize()
        ops.check_status()
        full = [x.clone() for x in (d, de, c, ce, p, pe, ts, tot)]
        assert plan(0) == 0
        torch.cuda.synchronize()
        assert all(torch.equal(a, b) for a, b in zip(full, (d, de, c, ce, p, pe, ts, tot)))

        def nonempty(seg, end):
            seg, end = seg.cpu().numpy(), end.cpu().numpy()
            keep = seg[:, 2] > 0
            return seg[keep], end[keep]

        for (dev_seg, dev_end), (h_seg, h_end) in (((d, de), host.dispatch), ((c, ce), host.combine),
                                                   ((p, pe), host.padding)):
            s, e = nonempty(dev_seg, dev_end)
            assert np.array_equal(s, h_seg) and np.array_equal(e, h_end)
        assert ts.cpu().tolist() == host.tile_start[rank].tolist()
        assert tot.cpu().tolist() == [int(host.send_rows[rank]), int(host.recv_rows[rank]),
                                      int(host.padding[0][:, 2].sum()), int(host.rows_grouped[rank])]


def test_push_rows_gathers_scatters_and_zeroes_locally():
    """ffm_p2p_push_rows with every destination on this GPU: gather through an index, run-wise scatter, zero rows,
    and the variant that reads the row total on the device."""
    torch.manual_seed(29)
    lib = _lib.load()
    W = 96
    src = torch.randn(50, W, device=DEV).bfloat16()
    index = torch.randint(0, 50 * 2, (40,), dtype=torch.int32, device=DEV)          # flat slots, two per token
    dst0 = torch.full((64, W), 3.0, device=DEV).bfloat16()
    dst1 = torch.full((64, W), 3.0, device=DEV).bfloat16()
    seg = torch.tensor([[0, 10, 7, 0], [7, 0, 0, 1], [7, 5, 20, 1], [27, 40, 13, 0]], dtype=torch.int64, device=DEV)
    end = torch.cumsum(seg[:, 2], 0)
    import ctypes
    bases = (ctypes.c_void_p * 2)(dst0.data_ptr(), dst1.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.ffm_p2p_push_rows(src.data_ptr(), index.data_ptr(), 2, W * 2, seg.data_ptr(), end.data_ptr(), 4, 40,
                                 bases, 2, stream) == 0
    torch.cuda.synchronize()
    rows = src[(index // 2).long()]
    ref0, ref1 = torch.full_like(dst0, 3.0), torch.full_like(dst1, 3.0)
    ref0[10:17] = rows[0:7]
    ref1[5:25] = rows[7:27]
    ref0[40:53] = rows[27:40]
    assert torch.equal(dst0, ref0) and torch.equal(dst1, ref1)
    # zeroing, with the total read on the device
    zseg = torch.tensor([[0, 60, 4, 1]], dtype=torch.int64, device=DEV)
    zend = torch.tensor([4], dtype=torch.int64, device=DEV)
    total = torch.tensor([4], dtype=torch.int64, device=DEV)
    assert lib.ffm_p2p_push_rows_dev(0, 0, 1, W * 2, zseg.data_ptr(), zend.data_ptr(), 1, total.data_ptr(), 64, bases, 2,
                                     stream) == 0
    torch.cuda.synchronize()
    ref1[60:64] = 0
    assert torch.equal(dst1, ref1) and torch.equal(dst0, ref0)


@pytest.mark.parametrize("activation", ["swiglu", "relu_squared"])
@pytest.mark.parametrize("counts,M,Nout,H", [([5, 0, 200, 128], 64, 64, 64), ([300, 17, 129, 64], 192, 320, 96),
                                             ([2048] * 8, 1024, 2048, 2048)])
def test_wgrad_with_glu_backward_passenger(counts, M, Nout, H, activation):
    """The weight-gradient GEMM that carries the GLU backward on extra warps equals the two separate kernels bit for
    bit, for both jobs. The passenger converts the rows below the end of the last group's tiles and leaves the rest
    of a (possibly much larger, worst-case sized) buffer alone."""
    torch.manual_seed(M + H)
    A, ts, row_expert, rows_cap = _grouped_case(counts, M)
    E = len(counts)
    Bx = torch.randn(rows_cap, Nout, device=DEV).bfloat16()
    Bx[row_expert == -1] = 0
    d_act = torch.randn(rows_cap + 37, H, device=DEV).bfloat16()       # the passenger has its own row count
    pre = torch.randn(rows_cap + 37, 2 * H, device=DEV).bfloat16()
    dW_ref = ops.grouped_gemm_wgrad(A, Bx, E, ts, scale=0.5)
    gU_ref = ops.glu_backward(d_act, pre, None, 1, activation)
    dW, gU = ops.grouped_gemm_wgrad_glu_backward(A, Bx, E, ts, d_act, pre, activation, scale=0.5)
    ops.check_status()
    assert torch.equal(dW, dW_ref)
    used = int(ts[-1]) * 128
    assert used <= rows_cap and torch.equal(gU[:used], gU_ref[:used])
    sentinel = torch.full_like(gU, 7.0)
    lib = _lib.load()
    rc = lib.ffm_grouped_gemm_wgrad_glu_backward(A.data_ptr(), Bx.data_ptr(), E, ts.data_ptr(), rows_cap, M, Nout, 0.5,
                                                 dW.data_ptr(), d_act.data_ptr(), pre.data_ptr(), d_act.shape[0], H,
                                                 _lib.ACTIVATION[activation], sentinel.data_ptr(),
                                                 ops.status_tensor(A.device).data_ptr(), ops._stream())
    assert rc == 0
    ops.check_status()
    assert torch.equal(sentinel[:used], gU_ref[:used]) and (sentinel[used:] == 7.0).all()


@pytest.mark.parametrize("activation", ["swiglu", "geglu", "relu_squared", "geglu_erf"])
@pytest.mark.parametrize("counts,K,H", [([5, 0, 200, 128], 64, 64), ([300, 17, 129, 64, 1, 0, 77, 256], 128, 320),
                                        ([2048] * 8, 1024, 2048)])
def test_dact_gemm_with_fused_glu_backward(counts, K, H, activation):
    """The dAct GEMM whose epilogue runs the GLU backward equals the dAct GEMM followed by the GLU backward kernel, bit
    for bit, on every row of the groups' tiles (ragged groups, empty groups, H not a multiple of the 256-column tile),
    also with a row buffer much larger than the rows in use, and for a dense (one group, ragged row count) call."""
    torch.manual_seed(K + H)
    gY, ts, row_expert, rows_cap = _grouped_case(counts, K)
    E = len(counts)
    Wd = (torch.randn(E, K, H, device=DEV) * 0.05).bfloat16()
    pre = torch.randn(rows_cap, 2 * H, device=DEV).bfloat16()
    used = int(ts[-1]) * 128
    want = ops.glu_backward(ops.grouped_gemm(gY, Wd, _lib.B_NMAJOR, E, ts, K, H), pre, ts, E, activation)
    got = ops.grouped_gemm_dact_glu_backward(gY, Wd, E, ts, K, H, pre, activation)
    ops.check_status()
    assert torch.equal(got[:used], want[:used])
    # worst-case sized buffers: three times the rows, only the groups' tiles are touched
    big_gY = torch.cat([gY, torch.randn(2 * rows_cap, K, device=DEV).bfloat16()])
    big_pre = torch.cat([pre, torch.randn(2 * rows_cap, 2 * H, device=DEV).bfloat16()])
    got_big = ops.grouped_gemm_dact_glu_backward(big_gY, Wd, E, ts, K, H, big_pre, activation)
    assert torch.equal(got_big[:used], want[:used])
    # dense, one group, a row count that is not a multiple of the tile height
    n = min(rows_cap, 333)
    dense_want = ops.glu_backward(ops.grouped_gemm(gY[:n].contiguous(), Wd[:1], _lib.B_NMAJOR, 1, None, K, H),
                                  pre[:n].contiguous(), None, 1, activation)
    dense_got = ops.grouped_gemm_dact_glu_backward(gY[:n].contiguous(), Wd[:1], 1, None, K, H, pre[:n].contiguous(),
                                                   activation)
    ops.check_status()
    assert torch.equal(dense_got, dense_want)


def test_kernel_timer_merges_overlapping_launches():
    """KernelTimer.union_ms counts the time two launches on different streams overlap once; the plain sum counts it
    twice."""
    timer = ops.KernelTimer()
    side = torch.cuda.Stream()
    x = torch.zeros(1 << 24, device=DEV)
    ops.set_timer(timer)
    try:
        with ops._Launch("a", 0):
            torch.cuda._sleep(2_000_000)
        with torch.cuda.stream(side):
            with ops._Launch("b", 0):
                torch.cuda._sleep(2_000_000)
        with ops._Launch("c", 0):
            x.add_(1.0)
    finally:
        ops.set_timer(None)
    torch.cuda.synchronize()
    totals = timer.totals_ms()
    both = timer.union_ms(("a", "b"))
    assert max(totals["a"][1], totals["b"][1]) <= both + 1e-3
    assert both < totals["a"][1] + totals["b"][1]          # the two sleeps ran at the same time
    assert abs(timer.union_ms(("a", "b"), exclude=("b",)) - totals["a"][1]) < 1e-3
    assert timer.union_ms(("missing",)) == 0.0
