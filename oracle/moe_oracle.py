"""CPU oracle for the fused MoE layer — TEST INFRASTRUCTURE ONLY.

A plain-torch (CPU) restatement of the algorithm of the reference project FlashFusedMoE
(src/flashfusemoe/...), written on unpadded per-expert rows. Only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py may import this module; the product package never does.

Parity status: PINNED. `oracle/pin_against_reference.py` runs the unmodified reference on CPU (its Triton
kernels through TRITON_INTERPRET=1) and checks this file against it; the same script writes the golden
vectors under tests/golden/ that the CPU test-suite replays.

Rounding points follow the reference's CUDA path in the compute dtype `dtype` (bf16 on the GPU, fp32 for the
CPU configuration): every matmul accumulates in fp32 and rounds its output to `dtype`; activations and
reductions are computed in fp32 from the rounded values and rounded again on store.
"""

import math

import torch

WEIGHT_EPS = 1e-6  # fused_moe.py:29


def _acc(dtype):
    return torch.float64 if dtype == torch.float64 else torch.float32


def mm(a, b, dtype):
    """a @ b with wide accumulation, output rounded to the compute dtype (torch.bmm / `@` in the reference)."""
    acc = _acc(dtype)
    return (a.to(acc) @ b.to(acc)).to(dtype)


# ----------------------------------------------------------------------------------------------
# Routing
# ----------------------------------------------------------------------------------------------

def gate_logits(hidden_c, gate_c, dtype):
    """fused_moe.py:334 — logits = hidden @ gate^T in the compute dtype."""
    return mm(hidden_c, gate_c.T, dtype)


def lowest_index_topk(sel, k):
    """kernels/fused_topk.py:53-70 — iterative argmax; ties go to the lowest index; descending order."""
    N, E = sel.shape
    sel = sel.clone()
    ar = torch.arange(E).expand(N, E)
    cols = []
    rows = torch.arange(N)
    for _ in range(k):
        m = sel.max(dim=1, keepdim=True).values
        idx = torch.where(sel == m, ar, torch.full_like(ar, E)).min(dim=1).values
        cols.append(idx)
        sel[rows, idx] = float("-inf")
    return torch.stack(cols, dim=1)


def group_limited_mask(sel, top_k, n_group, topk_group):
    """fused_moe.py:203-245 — eligibility mask [N, E]: the topk_group groups (of E / n_group contiguous experts)
    with the best sum of their top (top_k // topk_group) selection values (the maximum when that count is 1 or
    larger than the group) stay eligible. Ties between groups go to the lower group index."""
    N, E = sel.shape
    epg = E // n_group
    grouped = sel.view(N, n_group, epg)
    per_group = top_k // topk_group
    if 1 < per_group <= epg:
        gscore = grouped.topk(per_group, dim=-1).values.sum(dim=-1)
    else:
        gscore = grouped.max(dim=-1).values
    gidx = lowest_index_topk(gscore, topk_group)
    gmask = torch.zeros(N, n_group, dtype=torch.bool)
    gmask.scatter_(1, gidx, True)
    return gmask.unsqueeze(-1).expand(-1, -1, epg).reshape(N, E)


def route(logits, gating, top_k, expert_bias=None, scoring_factor=None, pre_softmax=False, n_group=None,
          topk_group=None):
    """Top-k weights and indices.

    Without bias: kernels/fused_topk.py:31-136 (the CUDA fast path, fused_moe.py:139-142).
    With expert_bias: fused_moe.py:165-179 (softmax) and :181-195 (sigmoid): selection on the biased values,
    weights from the unbiased ones. pre_softmax: fused_moe.py:146-162. n_group / topk_group: :203-251.
    Ties are resolved by the lowest-index rule everywhere.
    """
    lg = logits.float()
    if gating == "softmax":
        val = torch.softmax(lg, dim=-1) if pre_softmax else lg
    elif gating == "sigmoid":
        val = torch.sigmoid(lg)
    else:
        raise ValueError(f"Unknown gating: {gating}")
    sel = val if expert_bias is None else val + expert_bias.float().unsqueeze(0)
    if n_group is not None and topk_group is not None:
        sel = sel.masked_fill(~group_limited_mask(sel, top_k, n_group, topk_group), float("-inf"))
    idx = lowest_index_topk(sel, top_k)
    picked = val.gather(1, idx)
    if gating == "softmax" and not pre_softmax:
        w = torch.softmax(picked, dim=-1)
    else:
        w = picked / (picked.sum(dim=-1, keepdim=True) + WEIGHT_EPS)
    if scoring_factor is not None:
        w = w * (scoring_factor / top_k)  # fused_moe.py:197-198
    return w, idx


def sort_metadata(topk_idx, E):
    """fused_moe.py:344-348 — stable sort of the flat slots by expert, counts and starts."""
    flat = topk_idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E)
    starts = torch.zeros(E + 1, dtype=torch.long)
    starts[1:] = torch.cumsum(counts, 0)
    return order, counts, starts


def grouped_layout(topk_idx, E, tile=128, align=256):
    """The product's grouped-row layout: the stable order above with every expert segment starting on a
    multiple of `align` rows; tile_start counts `tile`-row tiles. Returns (tile_start[E+1], pos[T],
    src[rows_cap])."""
    flat = topk_idx.reshape(-1)
    T = flat.numel()
    order, counts, starts = sort_metadata(topk_idx, E)
    tiles = ((counts + align - 1) // align) * (align // tile)
    tile_start = torch.zeros(E + 1, dtype=torch.long)
    tile_start[1:] = torch.cumsum(tiles, 0)
    rank = torch.arange(T) - starts[flat[order]]
    pos = torch.empty(T, dtype=torch.long)
    pos[order] = tile_start[flat[order]] * tile + rank
    rows_cap = ((T + (align - 1) * E) // align) * align
    src = torch.full((rows_cap,), -1, dtype=torch.long)
    src[pos] = torch.arange(T)
    return tile_start, pos, src


def losses(logits, topk_w, topk_idx, gating, aux_loss_coeff, z_loss_coeff):
    """fused_moe.py:1175-1194. Differentiable w.r.t. `logits` / `topk_w` when they carry autograd history."""
    N, E = logits.shape
    out = {}
    flat = topk_idx.reshape(-1)
    tpe = torch.bincount(flat, minlength=E).float()
    if aux_loss_coeff > 0.0:
        f = tpe / N
        if gating == "softmax":
            P = torch.zeros(E, dtype=torch.float32).scatter_add(0, flat, topk_w.reshape(-1).float()) / N
        else:
            P = torch.sigmoid(logits.float()).mean(dim=0)
        out["aux_loss"] = aux_loss_coeff * E * (f * P).sum()
    if z_loss_coeff > 0.0:
        out["z_loss"] = z_loss_coeff * torch.logsumexp(logits.float(), dim=-1).square().mean()
    return out


# ----------------------------------------------------------------------------------------------
# GLU activations (kernels/activations.py:28-142)
# ----------------------------------------------------------------------------------------------

_C = 0.7978845608028654


def _tanh_ref(x):
    return 2.0 * torch.sigmoid(2.0 * x) - 1.0  # activations.py:20-22


def glu_forward(x, activation, dtype):
    """x [M, 2H] in compute dtype -> act(gate) * up, computed in fp32, stored in compute dtype."""
    H = x.shape[-1] // 2
    g, u = x[..., :H].float(), x[..., H:].float()
    if activation == "swiglu":
        r = g * torch.sigmoid(g) * u
    elif activation == "geglu":
        r = 0.5 * g * (1.0 + _tanh_ref(_C * (g + 0.044715 * g * g * g))) * u
    elif activation == "relu_squared":
        rg = torch.clamp(g, min=0.0)
        r = rg * rg * u
    elif activation == "geglu_erf":  # nn.py:38-39, shared expert of the non-EP layer
        r = torch.nn.functional.gelu(g) * u
    else:
        raise ValueError(f"Unknown activation: {activation}")
    return r.to(dtype)


def glu_backward(ga, x, activation, dtype):
    """activations.py:78-142: returns [M, 2H] = (d gate | d up)."""
    H = x.shape[-1] // 2
    g, u, ga = x[..., :H].float(), x[..., H:].float(), ga.float()
    if activation == "swiglu":
        s = torch.sigmoid(g)
        du = ga * (g * s)
        dg = ga * u * (s * (1.0 + g * (1.0 - s)))
    elif activation == "geglu":
        inner = _C * (g + 0.044715 * g * g * g)
        th = _tanh_ref(inner)
        du = ga * (0.5 * g * (1.0 + th))
        dg = ga * u * (0.5 * (1.0 + th) + 0.5 * g * (1.0 - th * th) * _C * (1.0 + 3.0 * 0.044715 * g * g))
    elif activation == "relu_squared":
        rg = torch.clamp(g, min=0.0)
        du = ga * rg * rg
        dg = ga * u * 2.0 * rg
    elif activation == "geglu_erf":
        cdf = 0.5 * (1.0 + torch.erf(g / math.sqrt(2.0)))
        pdf = torch.exp(-0.5 * g * g) / math.sqrt(2.0 * math.pi)
        du = ga * g * cdf
        dg = ga * u * (cdf + g * pdf)
    else:
        raise ValueError(f"Unknown activation: {activation}")
    return torch.cat([dg, du], dim=-1).to(dtype)


# ----------------------------------------------------------------------------------------------
# Full layer, forward and hand-written backward (fused_moe.py:308-595), on unpadded rows
# ----------------------------------------------------------------------------------------------

def fused_moe_forward(hidden, gate_w, w_up, w_down, top_k, activation="swiglu", gating="softmax",
                      aux_loss_coeff=0.0, z_loss_coeff=0.0, dtype=None, expert_bias=None, scoring_factor=None,
                      pre_softmax=False, n_group=None, topk_group=None, capacity_factor=None):
    """Returns a dict with the output, the losses and every intermediate the backward needs."""
    dtype = dtype or hidden.dtype
    h = hidden.to(dtype)
    g = gate_w.to(dtype)
    wu = w_up.to(dtype)
    wd = w_down.to(dtype)
    N, D = h.shape
    E = g.shape[0]
    logits = gate_logits(h, g, dtype)
    topk_w, topk_idx = route(logits, gating, top_k, expert_bias, scoring_factor, pre_softmax, n_group, topk_group)
    ls = losses(logits, topk_w, topk_idx, gating, aux_loss_coeff, z_loss_coeff)  # before any dropping (:1160-1194)
    order, counts, starts = sort_metadata(topk_idx, E)
    T = N * top_k
    keep = torch.ones(N, top_k)
    if capacity_factor is not None:
        # fused_moe.py:351-390: first-come capacity per expert, dropped weights zeroed, the rest renormalised
        capacity = max(int((N / E) * capacity_factor), top_k)
        rank_sorted = torch.arange(T) - starts[topk_idx.reshape(-1)[order]]
        rank = torch.empty(T, dtype=torch.long)
        rank[order] = rank_sorted
        keep = (rank < capacity).view(N, top_k).float()
        topk_w = topk_w * keep
        wsum = topk_w.sum(dim=-1, keepdim=True)
        topk_w = topk_w / (wsum + (1.0 - (wsum > 0).float()))
    tok = order // top_k                     # token of each sorted row
    xs = h[tok]                              # [T, D]   (fused_routing_scatter, moe_ops.py:53-106)
    up = torch.empty(T, wu.shape[1], dtype=dtype)
    down = torch.empty(T, D, dtype=dtype)
    act = torch.empty(T, wu.shape[1] // 2, dtype=dtype)
    for e in range(E):
        a, b = int(starts[e]), int(starts[e + 1])
        if a == b:
            continue
        up[a:b] = mm(xs[a:b], wu[e].T, dtype)                    # fused_moe.py:435
        act[a:b] = glu_forward(up[a:b], activation, dtype)      # :438
        down[a:b] = mm(act[a:b], wd[e].T, dtype)                # :441
    flat_w = topk_w.to(dtype).reshape(-1)                       # :412
    inv = torch.empty(T, dtype=torch.long)
    inv[order] = torch.arange(T)                                # sorted row of each flat slot
    gathered = down[inv].float() * flat_w.float().unsqueeze(-1)  # moe_ops.py:190-199
    out = gathered.view(N, top_k, D).sum(1).to(dtype)
    return dict(out=out, losses=ls, keep=keep, logits=logits, topk_w=topk_w, topk_idx=topk_idx, order=order, counts=counts,
                starts=starts, inv=inv, xs=xs, up=up, act=act, down=down, flat_w=flat_w,
                h=h, g=g, wu=wu, wd=wd, dtype=dtype, activation=activation, gating=gating, top_k=top_k,
                aux_loss_coeff=aux_loss_coeff, z_loss_coeff=z_loss_coeff)


def fused_moe_backward(fw, grad_out, grad_aux=1.0, grad_z=1.0, aux_loss_grad="analytic"):
    """Gradients (dH, dGate, dW_up, dW_down) of  <out, grad_out> + grad_aux * aux_loss + grad_z * z_loss.

    The routed part follows the reference's hand-written backward (fused_moe.py:527-591). The loss terms are
    what torch autograd produces for the reference's loss block (fused_moe.py:1165-1194) on its CPU path;
    aux_loss_grad="reference_cuda" drops the softmax-gating aux term, which on the reference's CUDA fast path
    has no autograd history (kernels/fused_topk.py:161-162 allocates the weights with torch.empty).
    """
    dtype = fw["dtype"]
    h, g, wu, wd = fw["h"], fw["g"], fw["wu"], fw["wd"]
    N, D = h.shape
    E = g.shape[0]
    k = fw["top_k"]
    T = N * k
    go = grad_out.to(dtype).contiguous()
    order, starts, inv = fw["order"], fw["starts"], fw["inv"]
    tok = order // k
    topk_w, topk_idx = fw["topk_w"], fw["topk_idx"]
    # routing-weight gradient, fused_moe.py:533-535
    gathered_down = fw["down"][inv]
    go_exp = go.unsqueeze(1).expand(-1, k, -1).reshape(T, D)
    gw = (gathered_down.float() * go_exp.float()).sum(-1).view(N, k) * fw["keep"]  # dropped slots read a zero row
    # weighted scatter, moe_ops.py:258-288 (sorted rows)
    gyw = (go[tok].float() * fw["flat_w"][order].float().unsqueeze(-1)).to(dtype)
    d_act = torch.empty_like(fw["act"])
    d_up = torch.empty_like(fw["up"])
    dxs = torch.empty_like(fw["xs"])
    dwu = torch.zeros_like(wu)
    dwd = torch.zeros_like(wd)
    for e in range(E):
        a, b = int(starts[e]), int(starts[e + 1])
        if a == b:
            continue
        d_act[a:b] = mm(gyw[a:b], wd[e], dtype)                                     # :547
        d_up[a:b] = glu_backward(d_act[a:b], fw["up"][a:b], fw["activation"], dtype)  # :550
        dxs[a:b] = mm(d_up[a:b], wu[e], dtype)                                      # :553
        dwd[e] = mm(gyw[a:b].T, fw["act"][a:b], dtype)                              # :564
        dwu[e] = mm(d_up[a:b].T, fw["xs"][a:b], dtype)                              # :565
    dh = dxs[inv].float().view(N, k, D).sum(1).to(dtype)                            # :559
    # routing Jacobian, :573-584
    lg = fw["logits"].float()
    ac, zc = fw["aux_loss_coeff"], fw["z_loss_coeff"]
    counts_f = fw["counts"].float()
    gaux_e = grad_aux * ac * E * (counts_f / N) if ac > 0.0 else None   # d loss / d P_e
    if fw["gating"] == "softmax":
        gwx = gw
        if gaux_e is not None and aux_loss_grad == "analytic":
            gwx = gw + gaux_e[topk_idx] / N
        s = topk_w
        sg = (gwx * s).sum(-1, keepdim=True)
        gtl = s * (gwx - sg)
    else:
        sc = torch.sigmoid(lg)
        ts = sc.gather(1, topk_idx)
        gdw = (gw * topk_w).sum(-1, keepdim=True)
        gtl = (gw - gdw) / (ts.sum(-1, keepdim=True) + WEIGHT_EPS) * ts * (1.0 - ts)
    gl = torch.zeros(N, E, dtype=torch.float32).scatter_add(1, topk_idx, gtl)        # :587-588
    if fw["gating"] == "sigmoid" and gaux_e is not None:
        sc = torch.sigmoid(lg)
        gl = gl + gaux_e.unsqueeze(0) * sc * (1.0 - sc) / N
    if zc > 0.0:
        lse = torch.logsumexp(lg, dim=-1, keepdim=True)
        gl = gl + (grad_z * zc) * 2.0 * lse / N * torch.exp(lg - lse)
    glc = gl.to(dtype)                                                              # :589
    dh = (dh.float() + mm(glc, g, dtype).float()).to(dtype)                         # :590
    dgate = mm(glc.T, h, dtype)                                                     # :591
    return dict(dH=dh, dGate=dgate, dW_up=dwu, dW_down=dwd, gw=gw, gl=glc)


def glu_ffn(x, w_gate, w_up, w_down, activation, dtype):
    """Shared expert (nn.py:22-44, fused_moe.py:687-689)."""
    pre = torch.cat([mm(x, w_gate.T, dtype), mm(x, w_up.T, dtype)], dim=-1)
    return mm(glu_forward(pre, activation, dtype), w_down.T, dtype)
