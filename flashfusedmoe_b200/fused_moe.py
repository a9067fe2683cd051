"""Functional API of the fused MoE layer: gate -> top-k route -> GLU experts -> weighted combine.

Same call signature, return value and error behaviour as the reference's
`flashfusemoe.fused_moe` (src/flashfusemoe/fused_moe.py:1073-1246); every tensor operation runs in the
sm_100a kernels of libffmoe through `flashfusedmoe_b200.ops`. There is no CPU path and no other backend.

Semantics kept from the reference's CUDA path, with the places where this implementation chooses differently:
  * compute dtype is the autocast dtype if autocast is on, else the input dtype (fused_moe.py:93-97); only
    bfloat16 is implemented, anything else raises;
  * routing indices follow the Triton kernel's rule (lowest index wins ties) on bf16-rounded logits;
  * `aux_loss` and `z_loss` are returned as differentiable tensors whose gradients are folded analytically
    into the routing backward. On the reference's CUDA fast path the softmax-gating aux loss carries no
    gradient (fused_topk.py:161-162); `set_aux_loss_grad("reference_cuda")` reproduces that;
  * there is no padded [E, max_tokens, D] buffer, so no token is ever dropped by overflow.
    `max_tokens_per_expert` is only consulted when `allow_dropped_tokens=False` and the caller gave a value:
    the same RuntimeError("MoE routing overflow ...") is raised if an expert received more rows;
  * expert parallelism (ep_group / set_ep_group) keeps the reference's backward contract: `grad_hidden` holds
    the routing and shared-expert terms only and expert weight gradients are scaled by 1 / ep_size
    (fused_moe.py:956-966, :1001-1005).
"""

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib, ops
import os

from . import p2p
from .expert_parallel import all_to_all_rows, local_ids_from_counts

_WEIGHT_EPS = 1e-6

# Process-wide expert-parallel state (reference: fused_moe.py:67-69). One EP group per process.
_EP_GROUP = None
_EP_ACTIVE = False
_EP_BACKEND = "nccl"

# "analytic": aux loss back-propagates into the gate; "reference_cuda": constant for softmax gating.
_AUX_LOSS_GRAD = "analytic"

# Expert-parallel transport: "p2p" = peer stores into symmetric receive buffers (libffmoe kernels), "nccl" =
# torch.distributed all_to_all_single. Chosen by FFM_EP_TRANSPORT at import; p2p falls back to nccl per call when
# symmetric memory is unavailable or a receive would not fit.
_EP_TRANSPORT = os.environ.get("FFM_EP_TRANSPORT", "p2p")
# Measurement aid: when set, the row exchanges move nothing (the receive buffers keep whatever they held) while
# every other kernel of the step still runs; the difference against a normal step is the exposed exchange time.
_EP_DRY_EXCHANGE = False
# Overlap of HBM-bound kernels with the tensor-core GEMMs: the routing backward and the shared expert on side streams
# (they fill the gaps and tails between GEMMs), small kernels nothing waits for as side branches, and (without the
# fused GLU-backward epilogue below) the GLU backward as a passenger inside the dW_down GEMM's CTAs.
# FFM_OVERLAP=0 keeps one stream and separate kernels.
_OVERLAP = os.environ.get("FFM_OVERLAP", "1") != "0"
# GLU backward inside the dAct GEMM's epilogue (one launch, dAct never written, bit-identical to the two kernels): the
# default. FFM_FUSED_GLU_BACKWARD=0 goes back to a plain dAct GEMM with the GLU backward riding as a passenger in the
# dW_down GEMM (measured 2 % slower per layer step at d_model 1024, ffn_dim 4096 and 1 % at d_model 4096, ffn_dim 28672).
_FUSED_GLU_BWD = os.environ.get("FFM_FUSED_GLU_BACKWARD", "1") != "0"
# Peer-store transport only: move rows straight into the receivers' grouped layout (FFM_EP_DIRECT=0 keeps the
# contiguous-range exchange with a permute on either side, the layout the NCCL transport also uses).
_EP_DIRECT = os.environ.get("FFM_EP_DIRECT", "1") != "0"


# Expert GEMM precision of the single-GPU forward pass: "bf16", or "fp8" = e4m3 operands (activations quantised per
# row, weights per expert, fp32 accumulation, bf16 outputs) for the up- and down-projection. Opt-in; the
# backward pass always runs in bf16 on the saved bf16 tensors.
_EXPERT_GEMM = "bf16"
_fp8_weight_cache = {}


def set_expert_gemm_precision(mode):
    """"bf16" (default) or "fp8": run the routed experts' forward projections on e4m3 operands (single-GPU path,
    d_model and ffn_dim / 2 multiples of 128). Returns the previous mode."""
    global _EXPERT_GEMM
    if mode not in ("bf16", "fp8"):
        raise ValueError(f"unknown expert GEMM precision: {mode}")
    old, _EXPERT_GEMM = _EXPERT_GEMM, mode
    return old


def _quantized_weight(owner, w):
    """e4m3 copy of the weight tensor `w` [E, N, K] (bf16, possibly a cast copy of `owner`) with one scale per expert.
    Cached per owner, the caller's own weight tensor (normally an nn.Parameter): the entry is reused while that very
    object is alive, unmodified (same version counter) and still where it was; a weak reference drops the entry
    when the owner dies, so an address reused by another tensor can never hit a stale entry."""
    import weakref
    key = id(owner)
    hit = _fp8_weight_cache.get(key)
    if hit is not None and hit[0]() is owner and hit[1] == (owner._version, owner.data_ptr(), tuple(owner.shape)):
        return hit[2], hit[3]
    q, sc = ops.quantize_weight_e4m3(w)
    try:
        ref = weakref.ref(owner, lambda _r, k=key: _fp8_weight_cache.pop(k, None))
    except TypeError:
        return q, sc
    _fp8_weight_cache[key] = (ref, (owner._version, owner.data_ptr(), tuple(owner.shape)), q, sc)
    return q, sc


def _expert_ffn_forward(Xg, wu, wd, E, tile_start, D, H, activation, keep, small, owners=None):
    """Up-projection + GLU and down-projection of the routed experts over grouped rows: (act, pre, Y)."""
    if _EXPERT_GEMM == "fp8" and D % 128 == 0 and H % 128 == 0 and not small:
        xq, xs = ops.quantize_rows_e4m3(Xg)
        own_u, own_d = owners if owners is not None else (wu, wd)
        wuq, wus = _quantized_weight(own_u, wu)
        act, pre = ops.grouped_gemm_glu_fp8(xq, xs, wuq, wus, E, tile_start, D, H, activation, want_preact=keep)
        aq, as_ = ops.quantize_rows_e4m3(act)
        wdq, wds = _quantized_weight(own_d, wd)
        Y = ops.grouped_gemm_fp8(aq, as_, wdq, wds, E, tile_start, H, D)
        return act, pre, Y
    act, pre = ops.grouped_gemm_glu(Xg, wu, wu.view(-1, D)[H:], 2 * H, E, tile_start, D, H, activation,
                                    want_preact=keep, **small)
    Y = ops.grouped_gemm(act, wd, _lib.B_KMAJOR, E, tile_start, H, D, **small)
    return act, pre, Y


def set_ep_dry_exchange(enable):
    """Benchmark switch: skip the payload of the expert-parallel exchanges (results are then meaningless). In
    host-sync-free mode the row kernels then move local rows only and every barrier still runs; the host-planned
    path skips its exchange kernels altogether."""
    global _EP_DRY_EXCHANGE
    _EP_DRY_EXCHANGE = bool(enable)
    if not enable:
        _lib.load().ffm_p2p_set_local_only(-1)

_side_streams = {}
_dense_tile_start = {}
# Backward exchanges issued so far per process group: picks the receive region of the next one (see _backward_region).
_bwd_exchanges = {}


def set_aux_loss_grad(mode):
    """Choose how the load-balance loss back-propagates: "analytic" (default) or "reference_cuda"."""
    global _AUX_LOSS_GRAD
    if mode not in ("analytic", "reference_cuda"):
        raise ValueError(f"unknown aux loss gradient mode: {mode}")
    _AUX_LOSS_GRAD = mode


def _get_side_stream(name, priority=0):
    idx = torch.cuda.current_device()
    key = (idx, name)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=idx, priority=priority)
    return _side_streams[key]


def _fork_small(like):
    """(current stream, side stream for small kernels) with the side stream ordered after what the current one holds,
    or (None, None) when overlap is off or the data is not on a GPU. Work issued on the side stream is a parallel
    branch of a captured step and runs beside the GEMMs instead of between them; close with _join_small."""
    if not _OVERLAP or not like.is_cuda:
        return None, None
    cur = torch.cuda.current_stream()
    side = _get_side_stream("small")
    fork = torch.cuda.Event()
    fork.record(cur)
    side.wait_event(fork)
    return cur, side


def _join_small(cur, side, *made_on_side):
    """The current stream waits for the side stream; tensors allocated there are handed over to the current one."""
    done = torch.cuda.Event()
    done.record(side)
    cur.wait_event(done)
    for t in made_on_side:
        t.record_stream(cur)


def _get_compute_dtype(fallback_dtype):
    if torch.is_autocast_enabled("cuda"):
        return torch.get_autocast_dtype("cuda")
    return fallback_dtype


def _estimate_max_tokens(N, top_k, E):
    """The reference's static per-expert buffer bound (fused_moe.py:100-113): twice the balanced share,
    or every routed row when there are at most 4 rows per expert. Kept for callers that size buffers with it;
    the kernels here do not need it."""
    balanced = -(-N * top_k // E)
    bound = balanced + max(balanced, top_k)
    if N * top_k <= 4 * E:
        bound = N * top_k
    return bound


def _validate_inputs(hidden_states, gate_weight, w_up, w_down, top_k, activation, gating, ep_group=None):
    assert hidden_states.dim() == 2, f"hidden_states must be 2D [N, D], got {hidden_states.shape}"
    N, D = hidden_states.shape
    E = gate_weight.shape[0]
    E_w = w_up.shape[0]
    ffn_dim = w_up.shape[1]
    assert gate_weight.shape == (E, D), f"gate_weight must be [{E}, {D}], got {gate_weight.shape}"
    assert w_up.shape == (E_w, ffn_dim, D), f"w_up must be [{E_w}, {ffn_dim}, {D}], got {w_up.shape}"
    assert w_down.shape == (E_w, D, ffn_dim // 2), \
        f"w_down must be [{E_w}, {D}, {ffn_dim // 2}], got {w_down.shape}"
    if ep_group is not None:
        ep_size = torch.distributed.get_world_size(ep_group)
        assert E % ep_size == 0, f"n_experts ({E}) must be divisible by ep_size ({ep_size})"
        assert E_w == E // ep_size, f"With EP, w_up must have E/ep_size={E // ep_size} experts, got {E_w}"
    else:
        assert E_w == E, f"w_up must have {E} experts, got {E_w}"
    assert ffn_dim % 2 == 0, f"ffn_dim must be even, got {ffn_dim}"
    assert 1 <= top_k <= E, f"top_k must be in [1, {E}], got {top_k}"
    dev = hidden_states.device
    assert all(t.device == dev for t in [gate_weight, w_up, w_down]), "All tensors must be on same device"
    assert activation in ("swiglu", "geglu", "relu_squared"), f"Unknown activation: {activation}"
    assert gating in ("softmax", "sigmoid"), f"Unknown gating: {gating}"


@dataclass
class _Cfg:
    top_k: int
    activation: str
    gating: str
    aux_loss_coeff: float
    z_loss_coeff: float
    recompute: bool
    expert_bias: Optional[torch.Tensor]
    weight_scale: float
    aux_grad: str
    shared_activation: str = "swiglu"
    ep_group: object = None
    ep_full_input_grad: bool = False
    pre_softmax: bool = False
    n_group: int = 0
    topk_group: int = 0
    capacity: Optional[int] = None
    input_jitter: float = 0.0
    addend_ready: object = None   # CUDA event: the addend (shared expert output) was produced on another stream
    wants_grad: bool = True       # False: no input needs a gradient or grad mode is off (inference shortcuts apply)


def _to(t, dtype):
    t = t if t.dtype == dtype else t.to(dtype)
    return t if t.is_contiguous() else t.contiguous()


def _dense_ts(rows, device, split=1):
    """tile_start for dense rows treated as `split` consecutive groups of 128-row tiles (cached per size; a tiny
    host-to-device copy)."""
    key = (torch.device(device).index, int(rows), split)
    t = _dense_tile_start.get(key)
    if t is None:
        tiles = (rows + 127) // 128
        t = torch.tensor([tiles * i // split for i in range(split + 1)], dtype=torch.int32, device=device)
        _dense_tile_start[key] = t
    return t


def _route(h, g, cfg, training):
    """Routing kernels for one call. With input_jitter the logits see h * U(1 - j, 1 + j) in training, exactly as
    the reference draws it (fused_moe.py:329-332); everything downstream uses the clean h."""
    h_route = h
    if cfg.input_jitter > 0.0 and training:
        noise = torch.empty_like(h).uniform_(1.0 - cfg.input_jitter, 1.0 + cfg.input_jitter)
        h_route = h * noise
    return ops.route_forward(h_route, g, cfg.top_k, cfg.gating, cfg.expert_bias, cfg.weight_scale,
                             pre_softmax=cfg.pre_softmax, n_group=cfg.n_group, topk_group=cfg.topk_group)


def _loss_tensors(routing, N, E, cfg):
    """aux = c E sum_e f_e P_e and z = c_z mean(lse^2) from the routing kernel's statistics (no host sync)."""
    aux = routing.stats[E + 1] * (cfg.aux_loss_coeff * E / (float(N) * float(N)))
    z = routing.stats[E] * (cfg.z_loss_coeff / float(N))
    return aux, z


def _loss_grads(routing, N, E, cfg, grad_aux, grad_z):
    """Device tensors fed to the routing backward: d loss / d P_e and d loss / d mean(lse^2)."""
    gaux = None
    if cfg.aux_loss_coeff > 0.0 and grad_aux is not None and (cfg.aux_grad == "analytic" or cfg.gating == "sigmoid"):
        gaux = routing.counts.to(torch.float32) * (grad_aux.to(torch.float32) * (cfg.aux_loss_coeff * E / float(N)))
    gz = None
    if cfg.z_loss_coeff > 0.0 and grad_z is not None:
        gz = (grad_z.to(torch.float32) * cfg.z_loss_coeff).reshape(1).contiguous()
    return gaux, gz


# ----------------------------------------------------------------------------------------------
# Dense GLU FFN (shared expert) on the same kernels: one group, stacked [gate; up] weights
# ----------------------------------------------------------------------------------------------

def _glu_ffn_forward(x, w_gate, w_up, w_down, activation, want_preact):
    Hs, D = w_gate.shape
    act, pre = ops.grouped_gemm_glu(x, w_gate, w_up, Hs, 1, None, D, Hs, activation, want_preact=want_preact)
    y = ops.grouped_gemm(act, w_down, _lib.B_KMAJOR, 1, None, Hs, D)
    return y, act, pre


def _glu_ffn_backward(go, x, act, pre, w_gate, w_up, w_down, activation):
    Hs, D = w_gate.shape
    fused = _FUSED_GLU_BWD and Hs % 64 == 0 and D % 64 == 0
    if fused:
        gU = ops.grouped_gemm_dact_glu_backward(go, w_down, 1, None, D, Hs, pre, activation)
    else:
        d_act = ops.grouped_gemm(go, w_down, _lib.B_NMAJOR, 1, None, D, Hs)
    ts = _dense_ts(x.shape[0], x.device)
    # [D, Hs] has few output tiles (32 CTA-pair tiles at D = 1024, Hs = 2048 for 74 pairs): split the token
    # dimension in two halves, each accumulated in fp32, and add the two bf16 results
    tiles = (x.shape[0] + 127) // 128
    split = 2 if tiles >= 64 and (D // 256) * ((Hs + 255) // 256) <= 40 else 1
    ts_down = _dense_ts(x.shape[0], x.device, split=2) if split == 2 else ts
    if fused:
        d_wdown = ops.grouped_gemm_wgrad(go, act, split, ts_down)
    elif _OVERLAP:
        # the GLU backward rides on extra warps of the dW_down GEMM, which does not depend on it
        d_wdown, gU = ops.grouped_gemm_wgrad_glu_backward(go, act, split, ts_down, d_act, pre, activation)
    else:
        gU = ops.glu_backward(d_act, pre, None, 1, activation)
        d_wdown = ops.grouped_gemm_wgrad(go, act, split, ts_down)
    cur, side = _fork_small(go)
    if side is None:
        d_wdown = d_wdown.sum(dim=0) if split == 2 else d_wdown[0]
        w_cat = torch.cat([w_gate, w_up], dim=0)
        dx = ops.grouped_gemm(gU, w_cat, _lib.B_NMAJOR, 1, None, 2 * Hs, D)
        d_wcat = ops.grouped_gemm_wgrad(gU, x, 1, ts)[0]
        return dx, d_wcat[:Hs], d_wcat[Hs:], d_wdown
    # the sum of the two partial products is needed only at the end: it runs as a side branch beside the next two
    # GEMMs. The stacked [gate; up] weights of the dX GEMM are copied on the current stream (the GEMM needs them next).
    parts = d_wdown
    parts.record_stream(side)  # freed below while the side stream may still read it
    with torch.cuda.stream(side):
        d_wdown = parts.sum(dim=0) if split == 2 else parts[0]
    w_cat = torch.cat([w_gate, w_up], dim=0)
    dx = ops.grouped_gemm(gU, w_cat, _lib.B_NMAJOR, 1, None, 2 * Hs, D)
    d_wcat = ops.grouped_gemm_wgrad(gU, x, 1, ts)[0]
    _join_small(cur, side, d_wdown)
    return dx, d_wcat[:Hs], d_wcat[Hs:], d_wdown


class _GLUFFNFunction(torch.autograd.Function):
    """y = act(x Wg^T) * (x Wu^T) Wd^T for the non-EP shared expert (reference: nn.py:22-44)."""

    @staticmethod
    def forward(ctx, x, w_gate, w_up, w_down, activation, dtype):
        xs = _to(x, dtype)
        wg, wu, wd = _to(w_gate, dtype), _to(w_up, dtype), _to(w_down, dtype)
        y, act, pre = _glu_ffn_forward(xs, wg, wu, wd, activation, want_preact=True)
        ctx.save_for_backward(xs, act, pre, wg, wu, wd)
        ctx.activation = activation
        ctx.in_dtypes = (x.dtype, w_gate.dtype, w_up.dtype, w_down.dtype)
        return y

    @staticmethod
    def backward(ctx, go):
        xs, act, pre, wg, wu, wd = ctx.saved_tensors
        go = _to(go, xs.dtype)
        dx, dwg, dwu, dwd = _glu_ffn_backward(go, xs, act, pre, wg, wu, wd, ctx.activation)
        dt = ctx.in_dtypes
        return dx.to(dt[0]), dwg.to(dt[1]), dwu.to(dt[2]), dwd.to(dt[3]), None, None


@torch.compiler.disable
def run_beside(fn, *args):
    """fn(*args) on the shared-expert side stream, ordered after the work already queued on the current stream.
    Returns (result, event recorded when it is done), or (fn(*args), None) when overlap is switched off. Autograd
    runs the backward of what fn recorded on that same stream, beside the routed experts' backward."""
    if not _OVERLAP or not args[0].is_cuda:
        return fn(*args), None
    side = _get_side_stream("shared", priority=-1)
    fork = torch.cuda.Event()
    fork.record()
    with torch.cuda.stream(side):
        side.wait_event(fork)
        out = fn(*args)
        done = torch.cuda.Event()
        done.record(side)
    return out, done


@torch.compiler.disable
def glu_ffn(x, w_gate, w_up, w_down, activation="swiglu"):
    """Dense GLU feed-forward on the library's GEMM kernels. x [N, D] -> [N, D]."""
    dtype = _require_bf16(_get_compute_dtype(x.dtype))
    return _GLUFFNFunction.apply(x, w_gate, w_up, w_down, activation, dtype)


def _require_bf16(dtype):
    if dtype != torch.bfloat16:
        raise NotImplementedError(
            f"flashfusedmoe_b200 computes in bfloat16 on sm_100a; got compute dtype {dtype}. Pass bf16 tensors "
            "or run under torch.autocast('cuda', dtype=torch.bfloat16).")
    return dtype


# ----------------------------------------------------------------------------------------------
# Single-GPU layer
# ----------------------------------------------------------------------------------------------

class _FusedMoEFunction(torch.autograd.Function):
    """Routed experts on one GPU, optionally with the layer's shared expert (sw_*: its gate, up and down weights):
    its forward GEMMs run on a side stream beside routing and permute and its output is added inside the combine
    kernel; its backward GEMMs start with the backward pass, beside the row kernels that the routed GEMMs wait for.
    Outputs: (out [N, D], aux_loss, z_loss, tokens_per_expert, dropped)."""

    @staticmethod
    def forward(ctx, hidden_states, gate_weight, w_up, w_down, addend, sw_gate, sw_up, sw_down, cfg, dtype):
        N, D = hidden_states.shape
        E = gate_weight.shape[0]
        H = w_up.shape[1] // 2
        k = cfg.top_k
        h = _to(hidden_states, dtype)
        g = _to(gate_weight, dtype)
        wu = _to(w_up, dtype)
        wd = _to(w_down, dtype)
        add = None if addend is None else _to(addend, dtype)
        need_grad = cfg.wants_grad and any(ctx.needs_input_grad[:8])
        has_shared = sw_gate is not None
        shared_ready = None
        if has_shared:
            assert add is None, "either an addend or shared expert weights"
            swg, swu, swd = _to(sw_gate, dtype), _to(sw_up, dtype), _to(sw_down, dtype)
            if _OVERLAP:
                side = _get_side_stream("shared", priority=-1)
                fork = torch.cuda.Event()
                fork.record()
                with torch.cuda.stream(side):
                    side.wait_event(fork)
                    add, s_act, s_pre = _glu_ffn_forward(h, swg, swu, swd, cfg.shared_activation, want_preact=need_grad)
                    shared_ready = torch.cuda.Event()
                    shared_ready.record(side)
            else:
                add, s_act, s_pre = _glu_ffn_forward(h, swg, swu, swd, cfg.shared_activation, want_preact=need_grad)

        routing = _route(h, g, cfg, hidden_states.requires_grad)
        cur, branch = (None, None) if cfg.capacity is not None else _fork_small(h)
        if branch is None:
            aux, z = _loss_tensors(routing, N, E, cfg)  # from the routing before any capacity dropping
            if cfg.capacity is not None:
                dropped = ops.route_apply_capacity(routing, cfg.capacity)
            else:
                dropped = torch.zeros(1, dtype=torch.int32, device=h.device)
        else:
            # three one-block kernels that nothing in the layer waits for: a side branch, joined before returning
            with torch.cuda.stream(branch):
                aux, z = _loss_tensors(routing, N, E, cfg)
                dropped = torch.zeros(1, dtype=torch.int32, device=h.device)
        # Without a backward pass nothing sums over the padding rows, so they are not zeroed -- except with capacity
        # dropping: a dropped slot keeps its grouped row (now a padding row) with weight 0, and 0 * (whatever the
        # GEMMs make of uninitialised memory, possibly NaN) would reach the output through the combine.
        Xg = ops.permute_rows(h, routing.src, routing.rows_cap, k,
                              zero_padding=need_grad or cfg.capacity is not None)
        keep = need_grad and not cfg.recompute
        # inference with few rows per expert (decode): one CTA per 128-row tile and no work on tiles without rows
        small = _small_m_kwargs(not need_grad and cfg.capacity is None and N * k < 128 * E, routing.counts)
        act, pre, Y = _expert_ffn_forward(Xg, wu, wd, E, routing.tile_start, D, H, cfg.activation, keep, small,
                                          owners=(w_up, w_down))
        if add is not None and cfg.addend_ready is not None:
            torch.cuda.current_stream().wait_event(cfg.addend_ready)
            add.record_stream(torch.cuda.current_stream())
        if shared_ready is not None:
            torch.cuda.current_stream().wait_event(shared_ready)
            add.record_stream(torch.cuda.current_stream())
        out = ops.combine_forward(Y, routing.pos, routing.topk_w, N, k, addend=add)
        if branch is not None:
            _join_small(cur, branch, aux, z, dropped)

        ctx.set_materialize_grads(False)
        ctx.cfg = cfg
        ctx.shape = (N, D, E, H)
        ctx.rows_cap = routing.rows_cap
        ctx.in_dtypes = (hidden_states.dtype, gate_weight.dtype, w_up.dtype, w_down.dtype,
                         None if addend is None else addend.dtype) + tuple(
                             None if w is None else w.dtype for w in (sw_gate, sw_up, sw_down))
        saved = [h, g, wu, wd, routing.topk_w, routing.topk_idx, routing.logits, routing.lse, routing.counts,
                 routing.tile_start, routing.pos, routing.src, Xg]
        if keep:
            saved += [pre, act, Y]
        ctx.kept = keep
        ctx.has_shared = has_shared and need_grad
        if ctx.has_shared:
            saved += [s_act, s_pre, swg, swu, swd]
        ctx.save_for_backward(*saved)
        counts = routing.counts
        ctx.mark_non_differentiable(counts, dropped)
        return out, aux, z, counts, dropped

    @staticmethod
    def backward(ctx, grad_out, grad_aux, grad_z, _grad_counts, _grad_dropped):
        cfg = ctx.cfg
        N, D, E, H = ctx.shape
        k = cfg.top_k
        saved = ctx.saved_tensors
        (h, g, wu, wd, topk_w, topk_idx, logits, lse, counts, tile_start, pos, src, Xg) = saved[:13]
        if ctx.kept:
            pre, act, Y = saved[13:16]
        else:
            # recompute the three large tensors with the same kernels: bit-identical to the forward pass
            act, pre = ops.grouped_gemm_glu(Xg, wu, wu.view(-1, D)[H:], 2 * H, E, tile_start, D, H, cfg.activation,
                                            want_preact=True)
            Y = ops.grouped_gemm(act, wd, _lib.B_KMAJOR, E, tile_start, H, D)
        routing = ops.Routing(topk_w, topk_idx, logits, lse, counts, tile_start, pos, src, None, ctx.rows_cap, k, E)
        if grad_out is None:
            grad_out = torch.zeros(N, D, dtype=h.dtype, device=h.device)
        go = _to(grad_out, h.dtype)  # also densifies expanded (stride-0) gradients

        shared_done = None
        fork_s = None
        if ctx.has_shared and _OVERLAP:
            fork_s = torch.cuda.Event()
            fork_s.record()
        # first in launch order: the routed GEMMs wait for it, the shared expert's (launched next) do not
        gYw, gw = ops.combine_backward(go, Y, topk_w, src, ctx.rows_cap, k)
        if ctx.has_shared:
            s_act, s_pre, swg, swu, swd = saved[-5:]
            if _OVERLAP:
                # the shared expert's backward depends on the output gradient alone: its GEMMs start with the backward
                # pass, beside combine_backward, and the routed GEMMs follow them
                side = _get_side_stream("shared", priority=-1)
                with torch.cuda.stream(side):
                    side.wait_event(fork_s)
                    s_dx, s_dwg, s_dwu, s_dwd = _glu_ffn_backward(go, h, s_act, s_pre, swg, swu, swd,
                                                                  cfg.shared_activation)
                    shared_done = torch.cuda.Event()
                    shared_done.record(side)
                go.record_stream(side)
            else:
                s_dx, s_dwg, s_dwu, s_dwd = _glu_ffn_backward(go, h, s_act, s_pre, swg, swu, swd, cfg.shared_activation)

        if _OVERLAP:
            # Two GEMMs never share an SM, so the GEMMs stay in one chain and each HBM-bound kernel is paired with
            # a GEMM that does not depend on it:
            #   main:  dAct GEMM with the GLU backward in its epilogue -> dW_down GEMM -> dX GEMM -> un-permute (+ routing
            #          term); with FFM_FUSED_GLU_BACKWARD=0: dAct GEMM -> dW_down GEMM carrying the GLU backward as passenger
            #   gemm:  (after dX) dW_up GEMM
            #   route: routing backward (fills the gaps between GEMMs)
            main = torch.cuda.current_stream()
            gemm = _get_side_stream("backward_gemm")
            route = _get_side_stream("backward_route")
            fork = torch.cuda.Event()
            fork.record(main)
            with torch.cuda.stream(route):
                route.wait_event(fork)
                gaux, gz = _loss_grads(routing, N, E, cfg, grad_aux, grad_z)
                dH_route, d_gate = ops.route_backward(gw, routing, gaux, gz, h, g, cfg.gating, dH=None)
                route_done = torch.cuda.Event()
                route_done.record(route)
            if _FUSED_GLU_BWD and H % 64 == 0 and D % 64 == 0:
                # dAct GEMM with the GLU backward in its epilogue, then the plain dW_down GEMM
                gU = ops.grouped_gemm_dact_glu_backward(gYw, wd, E, tile_start, D, H, pre, cfg.activation)
                d_wd = ops.grouped_gemm_wgrad(gYw, act, E, tile_start)
            else:
                d_act = ops.grouped_gemm(gYw, wd, _lib.B_NMAJOR, E, tile_start, D, H)
                # the GLU backward rides on extra warps of the dW_down GEMM (one launch)
                d_wd, gU = ops.grouped_gemm_wgrad_glu_backward(gYw, act, E, tile_start, d_act, pre, cfg.activation)
            dXg = ops.grouped_gemm(gU, wu, _lib.B_NMAJOR, E, tile_start, 2 * H, D)
            dx_done = torch.cuda.Event()
            dx_done.record(main)
            with torch.cuda.stream(gemm):
                gemm.wait_event(dx_done)
                d_wu = ops.grouped_gemm_wgrad(gU, Xg, E, tile_start)
                join = torch.cuda.Event()
                join.record(gemm)
            main.wait_event(route_done)
            dH = ops.combine_forward(dXg, pos, None, N, k, addend=dH_route)
            main.wait_event(join)
            for t_side in (dH_route, d_gate, d_wu):
                t_side.record_stream(main)  # allocated on a side stream, consumed on the main one from here on
        else:
            d_act = ops.grouped_gemm(gYw, wd, _lib.B_NMAJOR, E, tile_start, D, H)
            gU = ops.glu_backward(d_act, pre, tile_start, E, cfg.activation)
            dXg = ops.grouped_gemm(gU, wu, _lib.B_NMAJOR, E, tile_start, 2 * H, D)
            dH = ops.combine_forward(dXg, pos, None, N, k)
            d_wd = ops.grouped_gemm_wgrad(gYw, act, E, tile_start)
            d_wu = ops.grouped_gemm_wgrad(gU, Xg, E, tile_start)
            gaux, gz = _loss_grads(routing, N, E, cfg, grad_aux, grad_z)
            dH, d_gate = ops.route_backward(gw, routing, gaux, gz, h, g, cfg.gating, dH=dH)

        dt = ctx.in_dtypes
        d_add = None
        if dt[4] is not None and ctx.needs_input_grad[4]:
            d_add = go.to(dt[4])
        s_grads = (None, None, None)
        if ctx.has_shared:
            if shared_done is not None:
                cur_s = torch.cuda.current_stream()
                cur_s.wait_event(shared_done)
                for t_side in (s_dx, s_dwg, s_dwu, s_dwd):
                    t_side.record_stream(cur_s)
            dH = dH + s_dx
            s_grads = (s_dwg.to(dt[5]), s_dwu.to(dt[6]), s_dwd.to(dt[7]))
        return (dH.to(dt[0]), d_gate.to(dt[1]), d_wu.to(dt[2]), d_wd.to(dt[3]), d_add) + s_grads + (None, None)


# ----------------------------------------------------------------------------------------------
# Expert-parallel layer
# ----------------------------------------------------------------------------------------------

class _EPPlan:
    """Row counts of one expert-parallel call, identical on every rank: cnt[s][d] = rows rank s sends to rank d.
    Built from one all-gather of the per-expert counts and the call's only host synchronisation."""

    def __init__(self, counts, ep, e_local, group, row_bytes):
        self.group = group
        self.rank = torch.distributed.get_rank(group)
        self.ep = ep
        all_counts = torch.empty(ep, counts.numel(), dtype=counts.dtype, device=counts.device)
        torch.distributed.all_gather_into_tensor(all_counts, counts.contiguous(), group=group)
        self.recv_counts = all_counts[:, self.rank * e_local:(self.rank + 1) * e_local].to(torch.int64)  # [ep, E_local]
        # the host sync of the call: the [ep, E] count matrix and, in the same copy, the device status word (a bounded
        # wait that ran out in an earlier kernel must not go on to produce garbage silently)
        host = torch.cat([all_counts.reshape(-1), ops.status_tensor(counts.device).to(all_counts.dtype)]).cpu()
        ops.raise_on_status(host[-1], counts.device)
        C = host[:-1].view(ep, -1).numpy()                # [ep, E] rows rank s routes to expert e
        self.cnt = [[int(v) for v in row] for row in C.reshape(ep, ep, e_local).sum(-1)]
        self.cnt_t = [[self.cnt[d][s] for d in range(ep)] for s in range(ep)]
        self.send_splits = self.cnt[self.rank]
        self.recv_splits = [self.cnt[s][self.rank] for s in range(ep)]
        self.M = sum(self.recv_splits)
        # peer-store transport when the symmetric buffer can hold the largest receive of any rank, either direction
        self.px = None
        if _EP_TRANSPORT == "p2p" and p2p.available() and ep <= 16:
            worst = max(max(sum(self.cnt[s][d] for s in range(ep)) for d in range(ep)),
                        max(sum(self.cnt[s]) for s in range(ep)))
            need = 1 << max(20, (2 * (worst + 256 * e_local) * row_bytes - 1).bit_length())  # twice the worst case
            self.px = p2p.get_exchange(group, counts.device, need)
        # Row-granular tables: rows travel straight between the senders' expert-sorted order and the receivers'
        # grouped layout (p2p.SegmentPlan), so neither side runs a staging permute around the exchange.
        self.seg = None
        if self.px is not None and _EP_DIRECT:
            sp = p2p.SegmentPlan(C, e_local, self.rank)
            if self.px.fits(int(max(sp.rows_grouped.max(), sp.send_rows.max())), row_bytes):
                self.seg = sp
                r = self.rank
                self.rows_l = int(sp.rows_grouped[r])
                (self.d_seg, self.d_end, self.c_seg, self.c_end, self.p_seg, self.p_end, ts) = self.px.upload(
                    sp.dispatch[0], sp.dispatch[1], sp.combine[0], sp.combine[1], sp.padding[0], sp.padding[1],
                    sp.tile_start[r])
                self.ts_l = ts.to(torch.int32)
                self.remote_dispatch = int(sp.dispatch[0][sp.dispatch[0][:, 3] != r, 2].sum())
                self.remote_combine = int(sp.combine[0][sp.combine[0][:, 3] != r, 2].sum())

    def dispatch_grouped(self, src, src_index, index_div, region, zero_padding=True):
        """Sender order (or, with src_index, a gather from the token matrix) -> every receiver's grouped layout in
        `region`; returns this rank's grouped rows [rows_l, W] (a view of the region). The padding rows are zeroed
        unless the caller says nothing will sum over them (forward without gradients)."""
        px, sp = self.px, self.seg
        W = src.shape[1]
        rb = W * src.element_size()
        dry = _EP_DRY_EXCHANGE
        px.push_rows(src, src_index, index_div, rb, self.d_seg, self.d_end, len(sp.dispatch[0]),
                     int(sp.send_rows[self.rank]), region, remote_rows=self.remote_dispatch, dry=dry)
        if zero_padding:
            px.push_rows(None, None, 1, rb, self.p_seg, self.p_end, len(sp.padding[0]),
                         int(sp.padding[0][:, 2].sum()), region, name="zero_padding")
        px.barrier(dry=dry)
        return px.region_view(region, self.rows_l, W, src.dtype)

    def combine_grouped(self, grouped, region):
        """Grouped layout of this rank -> every origin's sender order in `region`; returns this rank's [T, W] view."""
        px, sp = self.px, self.seg
        W = grouped.shape[1]
        rb = W * grouped.element_size()
        dry = _EP_DRY_EXCHANGE
        px.push_rows(grouped, None, 1, rb, self.c_seg, self.c_end, len(sp.combine[0]),
                     int(sp.recv_rows[self.rank]), region, remote_rows=self.remote_combine, dry=dry)
        px.barrier(dry=dry)
        return px.region_view(region, int(sp.send_rows[self.rank]), W, grouped.dtype)

    def exchange(self, rows, reverse, region):
        """Dispatch direction (reverse=False: rows ordered by destination rank) or its inverse. The result may be a
        view of a receive region that the next exchange on the same region overwrites: copy it to keep it."""
        cnt = self.cnt_t if reverse else self.cnt
        if self.px is not None and self.px.fits(max(sum(cnt[s][d] for s in range(self.ep)) for d in range(self.ep)),
                                                rows.shape[1] * rows.element_size()):
            return self.px.exchange(rows, cnt, region, dry=_EP_DRY_EXCHANGE), True
        in_splits = cnt[self.rank]
        out_splits = [cnt[s][self.rank] for s in range(self.ep)]
        if _EP_DRY_EXCHANGE:
            return rows.new_zeros(sum(out_splits), rows.shape[1]), False
        ops.a2a_bytes_sent += (sum(in_splits) - in_splits[self.rank]) * rows.shape[1] * rows.element_size()
        with ops._Launch("all_to_all", 0):
            return all_to_all_rows(rows, out_splits, in_splits, self.group), False


# Host-sync-free expert parallelism: set_ep_static_forward(max_tokens_per_rank) declares, with the same value on
# every rank, the most tokens a rank passes per call. The expert-parallel layer (forward and backward, without latent
# projection) then sizes its buffers for the worst case (every routed row of every rank arriving at one rank), shares
# the counts and builds the exchange tables on the device, and never reads anything back: a call is a fixed launch
# sequence that a CUDA graph can capture and replay. Kernels only touch the rows in use (the persistent GEMM stops at
# the last real tile), so the worst-case sizes cost address space and memory, not time.
_EP_STATIC_TOKENS = None
_EP_STATIC_ROWS = None


def set_ep_static_forward(max_tokens_per_rank, max_recv_rows=None):
    """Enable (int, identical on every rank) or disable (None) host-sync-free expert parallelism: inference and
    training calls without latent projection then run without reading the routing counts on the host.

    max_recv_rows (optional, identical on every rank) bounds the routed rows a rank's experts may receive in one
    call, and with it the size of every buffer (default: the worst case, every routed row of every rank; the
    reference's own bound is twice the balanced load, fused_moe.py:100-113). If the routing of a call would exceed
    it on any rank, that call moves and computes nothing and sets device status 106 (raised by a later fused_moe()
    call or ops.check_status()): rows are never dropped silently and never stored past a buffer."""
    global _EP_STATIC_TOKENS, _EP_STATIC_ROWS
    _EP_STATIC_TOKENS = None if max_tokens_per_rank is None else int(max_tokens_per_rank)
    _EP_STATIC_ROWS = None if (max_recv_rows is None or max_tokens_per_rank is None) else int(max_recv_rows)


class _FusedMoEEPStaticFunction(torch.autograd.Function):
    """Expert-parallel layer without a host read: routing -> counts to every rank (peer stores) -> tables built on
    the device (ffm_p2p_plan) -> rows into the owners' grouped layouts -> grouped GEMMs over the worst-case buffer
    -> rows back -> weighted combine. The backward pass reuses the forward's device tables for its one exchange of
    the weighted output gradient (and the reverse exchange of cfg.ep_full_input_grad). Same results, bit for bit, as
    _FusedMoEEPFunction with the peer-store transport."""

    @staticmethod
    def forward(ctx, hidden_states, gate_weight, w_up, w_down, sw_gate, sw_up, sw_down, cfg, dtype):
        group = cfg.ep_group
        ep = torch.distributed.get_world_size(group)
        N, D = hidden_states.shape
        El = w_up.shape[0]
        E = ep * El
        H = w_up.shape[1] // 2
        k = cfg.top_k
        T = N * k
        if N > _EP_STATIC_TOKENS:
            raise RuntimeError(f"static expert-parallel mode was declared for at most {_EP_STATIC_TOKENS} tokens per "
                               f"rank, got {N}")
        has_shared = sw_gate is not None
        h, g, wu, wd = _to(hidden_states, dtype), _to(gate_weight, dtype), _to(w_up, dtype), _to(w_down, dtype)
        need_grad = cfg.wants_grad and any(ctx.needs_input_grad[:7])
        routing = _route(h, g, cfg, hidden_states.requires_grad)
        shared = None
        if has_shared:
            swg, swu, swd = _to(sw_gate, dtype), _to(sw_up, dtype), _to(sw_down, dtype)
            side = _get_side_stream("shared", priority=-1)
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(side):
                side.wait_event(ready)
                s_out, s_act, s_pre = _glu_ffn_forward(h, swg, swu, swd, cfg.shared_activation, want_preact=need_grad)
            shared_done = torch.cuda.Event()
            shared_done.record(side)
            shared = (s_out, s_act, s_pre, swg, swu, swd)
        rb = D * h.element_size()
        worst = ep * _EP_STATIC_TOKENS * k                       # every routed row of every rank lands on one rank
        bounded = _EP_STATIC_ROWS is not None and _EP_STATIC_ROWS < worst
        cap_rows = ((_EP_STATIC_ROWS if bounded else worst) + 256 * El + 255) // 256 * 256
        px = p2p.get_exchange(group, h.device, max(cap_rows, _EP_STATIC_TOKENS * k) * rb)
        C = px.share_counts(routing.counts)
        t = px.plan_dev(C, El, max_grouped_rows=cap_rows if bounded else 0)
        cpos, src_c = _compact_send_map(routing, T)
        tot = t["totals"]
        # measurement aid: with the dry switch on, the row kernels leave out every row bound for another GPU (local rows,
        # barriers and everything else still run)
        _lib.load().ffm_p2p_set_local_only(px.rank if _EP_DRY_EXCHANGE else -1)
        px.push_rows_dev(h, src_c, k, rb, t["dispatch"], t["dispatch_end"], tot[0:1], T, 0)
        if need_grad:
            # the weight-gradient GEMMs sum over whole 64-row blocks: the padding rows of the grouped layout are zeroed
            # (without a backward pass nothing sums over them, and a GEMM row only depends on its own input row)
            px.push_rows_dev(None, None, 1, rb, t["padding"], t["padding_end"], tot[2:3], 256 * El, 0,
                             name="zero_padding")
        px.barrier_dev()
        # The GEMMs and the combine read the received rows in place. The copies that the backward pass needs (the
        # regions are overwritten by the next call) are side branches: the copy of the grouped rows must be complete
        # before this rank signals the combine exchange (a peer that has passed that barrier may push the next call's
        # rows into region 0), the copy of the returned rows before it signals the next dispatch, i.e. before the
        # forward pass returns.
        Xg = px.region_view(0, cap_rows, D, h.dtype)
        Xg_saved = returned_saved = None
        cur, copier = _fork_small(h) if need_grad else (None, None)
        if need_grad and copier is None:
            Xg = Xg_saved = px.keep_rows_dev(Xg, tot[3:4], cap_rows)
        elif need_grad:
            with torch.cuda.stream(copier):
                Xg_saved = px.keep_rows_dev(Xg, tot[3:4], cap_rows)
        small = _small_m_kwargs(not need_grad and ep * _EP_STATIC_TOKENS * k < 128 * E, None)
        if small:
            small["valid_rows"] = C[:, px.rank * El:(px.rank + 1) * El].sum(0, dtype=torch.int32)
        act, pre = ops.grouped_gemm_glu(Xg, wu, wu.view(-1, D)[H:], 2 * H, El, t["tile_start"], D, H, cfg.activation,
                                        want_preact=need_grad, **small)
        Y = ops.grouped_gemm(act, wd, _lib.B_KMAJOR, El, t["tile_start"], H, D, **small)
        if copier is not None:
            _join_small(cur, copier, Xg_saved)
        px.push_rows_dev(Y, None, 1, rb, t["combine"], t["combine_end"], tot[1:2], cap_rows, 1)
        px.barrier_dev()
        returned = px.region_view(1, T, D, h.dtype)
        if need_grad and copier is None:
            returned = returned_saved = returned.clone()
        elif need_grad:
            cur, copier = _fork_small(h)
            with torch.cuda.stream(copier):
                returned_saved = returned.clone()
        if has_shared:
            torch.cuda.current_stream().wait_event(shared_done)
        out = ops.combine_forward(returned, cpos, routing.topk_w, N, k, addend=shared[0] if has_shared else None)
        if need_grad and copier is not None:
            _join_small(cur, copier, returned_saved)
        aux, z = _loss_tensors(routing, N, E, cfg)

        ctx.set_materialize_grads(False)
        ctx.cfg = cfg
        ctx.dims = (N, D, E, El, H, k, ep, cap_rows)
        ctx.has_shared = has_shared
        ctx.px = px
        ctx.in_dtypes = tuple(None if x is None else x.dtype for x in
                              (hidden_states, gate_weight, w_up, w_down, sw_gate, sw_up, sw_down))
        ctx.rows_cap = routing.rows_cap
        if need_grad:
            tensors = dict(h=h, g=g, wu=wu, wd=wd, topk_w=routing.topk_w, topk_idx=routing.topk_idx,
                           logits=routing.logits, lse=routing.lse, counts=routing.counts, src_c=src_c, cpos=cpos,
                           returned=returned_saved, Xg=Xg_saved, act=act, pre=pre, ts_l=t["tile_start"], totals=tot,
                           dispatch=t["dispatch"], dispatch_end=t["dispatch_end"], combine=t["combine"],
                           combine_end=t["combine_end"], padding=t["padding"], padding_end=t["padding_end"])
            if has_shared:
                tensors.update(s_act=shared[1], s_pre=shared[2], swg=shared[3], swu=shared[4], swd=shared[5])
            ctx.names = list(tensors)
            ctx.save_for_backward(*tensors.values())
        counts = routing.counts
        dropped = torch.zeros(1, dtype=torch.int32, device=h.device)
        ctx.mark_non_differentiable(counts, dropped)
        return out, aux, z, counts, dropped

    @staticmethod
    def backward(ctx, grad_out, grad_aux, grad_z, _grad_counts, _grad_dropped):
        cfg = ctx.cfg
        group = cfg.ep_group
        N, D, E, El, H, k, ep, cap_rows = ctx.dims
        px = ctx.px
        t = dict(zip(ctx.names, ctx.saved_tensors))
        h, g, wu, wd = t["h"], t["g"], t["wu"], t["wd"]
        T = N * k
        rb = D * h.element_size()
        tot = t["totals"]
        if grad_out is None:
            grad_out = torch.zeros(N, D, dtype=h.dtype, device=h.device)
        go = _to(grad_out, h.dtype)
        inv_ep = 1.0 / ep

        if ctx.has_shared:
            side = _get_side_stream("shared", priority=-1)
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(side):
                side.wait_event(ready)
                s_dx, s_dwg, s_dwu, s_dwd = _glu_ffn_backward(go, h, t["s_act"], t["s_pre"], t["swg"], t["swu"],
                                                              t["swd"], cfg.shared_activation)
            shared_done = torch.cuda.Event()
            shared_done.record(side)

        # routing-weight gradient and weighted output gradient in send order, then the one exchange of the backward
        # pass on a side stream while the routing backward runs on the main one
        gYw, gw = ops.combine_backward(go, t["returned"], t["topk_w"], t["src_c"], T, k)
        a2a = _get_side_stream("a2a")
        ready2 = torch.cuda.Event()
        ready2.record()
        region = _backward_region(group)
        _lib.load().ffm_p2p_set_local_only(px.rank if _EP_DRY_EXCHANGE else -1)
        with torch.cuda.stream(a2a):
            a2a.wait_event(ready2)
            px.push_rows_dev(gYw, None, 1, rb, t["dispatch"], t["dispatch_end"], tot[0:1], T, region)
            px.push_rows_dev(None, None, 1, rb, t["padding"], t["padding_end"], tot[2:3], 256 * El, region,
                             name="zero_padding")
            px.barrier_dev()
        a2a_done = torch.cuda.Event()
        a2a_done.record(a2a)
        gYw.record_stream(a2a)
        gYg = px.region_view(region, cap_rows, D, h.dtype)

        routing = ops.Routing(t["topk_w"], t["topk_idx"], t["logits"], t["lse"], t["counts"], None, None, None, None,
                              ctx.rows_cap, k, E)
        gaux, gz = _loss_grads(routing, N, E, cfg, grad_aux, grad_z)
        dH, d_gate = ops.route_backward(gw, routing, gaux, gz, h, g, cfg.gating, dH=None)

        torch.cuda.current_stream().wait_event(a2a_done)
        ts_l = t["ts_l"]
        if _FUSED_GLU_BWD and H % 64 == 0 and D % 64 == 0:
            gU = ops.grouped_gemm_dact_glu_backward(gYg, wd, El, ts_l, D, H, t["pre"], cfg.activation)
            d_wd = _grouped_wgrad(gYg, t["act"], El, ts_l, scale=inv_ep)
        else:
            d_act = ops.grouped_gemm(gYg, wd, _lib.B_NMAJOR, El, ts_l, D, H)
            if _OVERLAP:
                d_wd, gU = _grouped_wgrad(gYg, t["act"], El, ts_l, scale=inv_ep,
                                          passenger=(d_act, t["pre"], cfg.activation))
            else:
                gU = ops.glu_backward(d_act, t["pre"], ts_l, El, cfg.activation)
                d_wd = _grouped_wgrad(gYg, t["act"], El, ts_l, scale=inv_ep)
        d_wu = _grouped_wgrad(gU, t["Xg"], El, ts_l, scale=inv_ep)
        if cfg.ep_full_input_grad:
            dXg = ops.grouped_gemm(gU, wu, _lib.B_NMAJOR, El, ts_l, 2 * H, D)
            px.push_rows_dev(dXg, None, 1, rb, t["combine"], t["combine_end"], tot[1:2], cap_rows, 1)
            px.barrier_dev()
            d_send = px.region_view(1, T, D, h.dtype)
            dH = dH + ops.combine_forward(d_send, t["cpos"], None, N, k)
        s_grads = (None, None, None)
        if ctx.has_shared:
            torch.cuda.current_stream().wait_event(shared_done)
            dH = dH + s_dx
            s_grads = (s_dwg, s_dwu, s_dwd)
        dt = ctx.in_dtypes

        def cast(x, i):
            return None if x is None or dt[i] is None else x.to(dt[i])

        return (cast(dH, 0), cast(d_gate, 1), cast(d_wu, 2), cast(d_wd, 3), cast(s_grads[0], 4), cast(s_grads[1], 5),
                cast(s_grads[2], 6), None, None)


def _wgrad_split_factor(groups, M, n_out):
    """How many K ranges to split every group's weight-gradient GEMM into so that its output tiles fill the GPU: with
    few local experts (expert parallel over many ranks) groups x tiles falls below the 74 CTA pairs."""
    units = groups * ((M + 255) // 256) * ((n_out + 255) // 256)
    return 1 if units >= 56 else min(4, max(1, 74 // units))


def _split_tile_start(tile_start, S):
    """tile_start [groups + 1] -> [groups * S + 1]: every group's tile range cut into S ranges of whole tile pairs."""
    ts = tile_start.to(torch.int64)
    lo, pairs = ts[:-1], (ts[1:] - ts[:-1]) // 2
    cuts = torch.stack([lo + 2 * ((pairs * s) // S) for s in range(S)], dim=1).reshape(-1)
    return torch.cat([cuts, ts[-1:]]).to(torch.int32)


def _grouped_wgrad(A, B, groups, tile_start, scale=1.0, passenger=None):
    """ops.grouped_gemm_wgrad, split along K into partial products (summed afterwards) when the output is too small
    to occupy every SM. passenger = (d_act, preact, activation): the GLU backward rides in the same launch and the
    result is (dW, gU)."""
    S = _wgrad_split_factor(groups, A.shape[1], B.shape[1])
    ts = tile_start if S == 1 else _split_tile_start(tile_start, S)
    gU = None
    if passenger is not None:
        part, gU = ops.grouped_gemm_wgrad_glu_backward(A, B, groups * S, ts, passenger[0], passenger[1], passenger[2],
                                                       scale=scale)
    else:
        part = ops.grouped_gemm_wgrad(A, B, groups * S, ts, scale=scale)
    if S > 1:
        part = part.view(groups, S, A.shape[1], B.shape[1]).sum(dim=1, dtype=torch.float32).to(part.dtype)
    return part if passenger is None else (part, gU)


def _backward_region(group):
    """Receive region of the next backward exchange of `group`: regions 2 and 3 in turn.

    The rows a backward exchange delivers are read in place by that layer's GEMMs, after the exchange's flag barrier.
    A peer that has left the barrier may already push the next layer's gradient rows, and nothing orders that push
    after this rank's reads, so two consecutive backward exchanges must not share a region. With two regions a peer's
    push n + 2 (the next one into the same region) comes after it has seen this rank's signal n + 1, which this rank
    issues, in stream order, after the reads of exchange n. Every rank runs the same sequence of layers, so the
    count, and with it the region, agrees across the group."""
    key = id(group)
    n = _bwd_exchanges.get(key, 0)
    _bwd_exchanges[key] = n + 1
    return 2 + (n & 1)


def _small_m_kwargs(enabled, counts):
    """Arguments that make the grouped GEMMs use 128-row single-CTA tiles and skip tiles without valid rows."""
    if not enabled:
        return {}
    return dict(valid_rows=None if counts is None else counts.to(torch.int32), tile_rows=128)


def _compact_send_map(routing, T):
    """Send-buffer position of every flat slot: the grouped order with the 256-row padding squeezed out.
    Rows are expert-major, hence destination-rank-major (each rank owns a contiguous block of experts)."""
    return ops.compact_positions(routing, T)


class _FusedMoEEPFunction(torch.autograd.Function):
    """Expert-parallel layer: route -> all-to-all dispatch -> local grouped GEMMs -> all-to-all combine.

    Mirrors reference _FusedMoEEPAutograd (fused_moe.py:598-1022): shared expert on a high-priority side
    stream, optional latent projection around both exchanges, backward with one exchange of the weighted
    output gradient, no expert input gradient unless cfg.ep_full_input_grad.
    """

    @staticmethod
    def forward(ctx, hidden_states, gate_weight, w_up, w_down, sw_gate, sw_up, sw_down, lw_down, lw_up, cfg, dtype):
        group = cfg.ep_group
        ep = torch.distributed.get_world_size(group)
        N, D = hidden_states.shape
        El = w_up.shape[0]
        E = ep * El
        H = w_up.shape[1] // 2
        k = cfg.top_k
        T = N * k
        has_shared = sw_gate is not None
        has_latent = lw_down is not None
        h = _to(hidden_states, dtype)
        g = _to(gate_weight, dtype)
        wu = _to(w_up, dtype)
        wd = _to(w_down, dtype)
        need_grad = cfg.wants_grad and any(ctx.needs_input_grad[:9])

        routing = _route(h, g, cfg, hidden_states.requires_grad)

        # shared expert on a side stream: queued before the host waits for the split sizes
        shared = None
        if has_shared:
            swg, swu, swd = _to(sw_gate, dtype), _to(sw_up, dtype), _to(sw_down, dtype)
            side = _get_side_stream("shared", priority=-1)
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(side):
                side.wait_event(ready)
                s_out, s_act, s_pre = _glu_ffn_forward(h, swg, swu, swd, cfg.shared_activation, want_preact=need_grad)
            shared_done = torch.cuda.Event()
            shared_done.record(side)
            shared = (s_out, s_act, s_pre, swg, swu, swd)

        if has_latent:
            lwd, lwu = _to(lw_down, dtype), _to(lw_up, dtype)
            L = lwd.shape[0]
            disp = ops.grouped_gemm(h, lwd, _lib.B_KMAJOR, 1, None, D, L)   # [N, L]
        else:
            disp = h

        W_bytes = disp.shape[1] * disp.element_size()
        plan = _EPPlan(routing.counts, ep, El, group, max(W_bytes, D * 2))
        recv_counts, M = plan.recv_counts, plan.M
        cpos, src_c = _compact_send_map(routing, T)
        direct = plan.seg is not None
        pos_l = src_l = None
        recv_lat = None
        if direct:
            # rows are gathered from the token matrix and stored straight into the owners' grouped layouts
            rows_l = plan.rows_l
            ts_l = plan.ts_l
            recv = plan.dispatch_grouped(disp, src_c, k, 0, zero_padding=need_grad)   # [rows_l, W] grouped, region view
            if need_grad:
                recv = recv.clone()  # saved for backward; the region is overwritten by the next call
            if has_latent:
                recv_lat = recv
                recv = (ops.grouped_gemm(recv, lwu, _lib.B_KMAJOR, 1, None, L, D) if rows_l > 0
                        else recv.new_empty(0, D))
            Xg = recv
        else:
            send = ops.permute_rows(disp, src_c, T, k)
            recv, is_view = plan.exchange(send, False, 0)                          # [M, W]
            if is_view and has_latent and need_grad:
                recv = recv.clone()  # saved for the latent weight gradients
            if M > 0:
                local_ids = local_ids_from_counts(recv_counts, M).to(torch.int32)
                _, ts_l, pos_l, src_l, rows_l = ops.group_rows(local_ids, El)
            else:
                ts_l = None
                rows_l = 0
            if has_latent:
                recv_lat = recv
                recv = ops.grouped_gemm(recv, lwu, _lib.B_KMAJOR, 1, None, L, D) if M > 0 else recv.new_empty(0, D)
            Xg = ops.permute_rows(recv, src_l, rows_l, 1) if M > 0 else None
        if M > 0:
            small = _small_m_kwargs(not need_grad and M < 128 * El, None)
            if small:
                small["valid_rows"] = recv_counts.sum(0, dtype=torch.int32)
            act, pre = ops.grouped_gemm_glu(Xg, wu, wu.view(-1, D)[H:], 2 * H, El, ts_l, D, H, cfg.activation,
                                            want_preact=need_grad, **small)
            Y = ops.grouped_gemm(act, wd, _lib.B_KMAJOR, El, ts_l, H, D, **small)
            # direct: the grouped rows go back as they lie; otherwise back to arrival order [M, D] first
            local_out = Y if direct else ops.combine_forward(Y, pos_l, None, M, 1)
        else:
            Xg = act = pre = None
            local_out = h.new_empty(0, D)
        local_out_D = local_out
        if has_latent and M > 0:
            local_out = ops.grouped_gemm(local_out, lwd, _lib.B_KMAJOR, 1, None, D, L)
        elif has_latent:
            local_out = h.new_empty(0, L)
        if direct:
            returned, is_view = plan.combine_grouped(local_out, 1), True           # [T, W], send order
        else:
            returned, is_view = plan.exchange(local_out, True, 1)                  # [T, W], send order
        if is_view and need_grad:
            returned = returned.clone()  # saved for backward; the region is overwritten by the next call
        returned_lat = None
        if has_latent:
            returned_lat = returned
            returned = ops.grouped_gemm(returned, lwu, _lib.B_KMAJOR, 1, None, L, D)
        if has_shared:
            torch.cuda.current_stream().wait_event(shared_done)
        out = ops.combine_forward(returned, cpos, routing.topk_w, N, k, addend=shared[0] if has_shared else None)
        aux, z = _loss_tensors(routing, N, E, cfg)

        ctx.set_materialize_grads(False)
        ctx.cfg = cfg
        ctx.dims = (N, D, E, El, H, k, M, ep, rows_l)
        ctx.flags = (has_shared, has_latent, direct)
        ctx.plan = plan
        ctx.in_dtypes = tuple(None if t is None else t.dtype for t in
                              (hidden_states, gate_weight, w_up, w_down, sw_gate, sw_up, sw_down, lw_down, lw_up))
        ctx.routing_meta = (routing.rows_cap,)
        tensors = dict(h=h, g=g, wu=wu, wd=wd, topk_w=routing.topk_w, topk_idx=routing.topk_idx,
                       logits=routing.logits, lse=routing.lse, counts=routing.counts, src_c=src_c, cpos=cpos,
                       returned=returned, ts_l=ts_l, src_l=src_l, pos_l=pos_l, Xg=Xg, act=act, pre=pre)
        if has_shared:
            tensors.update(s_act=shared[1], s_pre=shared[2], swg=shared[3], swu=shared[4], swd=shared[5])
        if has_latent:
            tensors.update(lwd=lwd, lwu=lwu, recv_lat=recv_lat, returned_lat=returned_lat, local_out_D=local_out_D)
        ctx.names = [n for n, t in tensors.items() if t is not None]
        ctx.save_for_backward(*[tensors[n] for n in ctx.names])
        counts = routing.counts
        dropped = torch.zeros(1, dtype=torch.int32, device=h.device)
        ctx.mark_non_differentiable(counts, dropped)
        return out, aux, z, counts, dropped

    @staticmethod
    def backward(ctx, grad_out, grad_aux, grad_z, _grad_counts, _grad_dropped):
        cfg = ctx.cfg
        group = cfg.ep_group
        N, D, E, El, H, k, M, ep, rows_l = ctx.dims
        has_shared, has_latent, direct = ctx.flags
        plan = ctx.plan
        t = dict(zip(ctx.names, ctx.saved_tensors))
        h, g, wu, wd = t["h"], t["g"], t["wu"], t["wd"]
        T = N * k
        if grad_out is None:
            grad_out = torch.zeros(N, D, dtype=h.dtype, device=h.device)
        go = _to(grad_out, h.dtype)
        inv_ep = 1.0 / ep

        # shared expert backward on the side stream
        if has_shared:
            side = _get_side_stream("shared", priority=-1)
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(side):
                side.wait_event(ready)
                s_dx, s_dwg, s_dwu, s_dwd = _glu_ffn_backward(go, h, t["s_act"], t["s_pre"], t["swg"], t["swu"],
                                                              t["swd"], cfg.shared_activation)
            shared_done = torch.cuda.Event()
            shared_done.record(side)

        # routing-weight gradient and weighted output gradient, in send order (fused_moe.py:882-898)
        gYw, gw = ops.combine_backward(go, t["returned"], t["topk_w"], t["src_c"], T, k)
        if has_latent:
            L = t["lwd"].shape[0]
            send = ops.grouped_gemm(gYw, t["lwu"], _lib.B_NMAJOR, 1, None, D, L)
        else:
            send = gYw

        # exchange on a side stream, routing backward meanwhile on the main stream (:901-932)
        a2a = _get_side_stream("a2a")
        ready2 = torch.cuda.Event()
        ready2.record()
        region = _backward_region(group)
        with torch.cuda.stream(a2a):
            a2a.wait_event(ready2)
            if direct:
                recv_grad, grad_is_view = plan.dispatch_grouped(send, None, 1, region), True   # grouped [rows_l, W]
            else:
                recv_grad, grad_is_view = plan.exchange(send, False, region)
        a2a_done = torch.cuda.Event()
        a2a_done.record(a2a)
        send.record_stream(a2a)

        routing = ops.Routing(t["topk_w"], t["topk_idx"], t["logits"], t["lse"], t["counts"], None, None, None, None,
                              ctx.routing_meta[0], k, E)
        gaux, gz = _loss_grads(routing, N, E, cfg, grad_aux, grad_z)
        dH, d_gate = ops.route_backward(gw, routing, gaux, gz, h, g, cfg.gating, dH=None)

        torch.cuda.current_stream().wait_event(a2a_done)
        if not grad_is_view:
            recv_grad.record_stream(torch.cuda.current_stream())
        d_lwd = d_lwu = None
        if has_latent:
            recv_grad_lat = recv_grad
            recv_grad = (ops.grouped_gemm(recv_grad_lat, t["lwu"], _lib.B_KMAJOR, 1, None, L, D)
                         if M > 0 else recv_grad.new_empty(0, D))
        if M > 0:
            gYg = recv_grad if direct else ops.permute_rows(recv_grad, t["src_l"], rows_l, 1)
            if _FUSED_GLU_BWD and H % 64 == 0 and D % 64 == 0:
                gU = ops.grouped_gemm_dact_glu_backward(gYg, wd, El, t["ts_l"], D, H, t["pre"], cfg.activation)
                d_wd = _grouped_wgrad(gYg, t["act"], El, t["ts_l"], scale=inv_ep)
            elif _OVERLAP:
                # the down-projection weight gradient does not need the GLU backward: it carries it as a passenger
                d_act = ops.grouped_gemm(gYg, wd, _lib.B_NMAJOR, El, t["ts_l"], D, H)
                d_wd, gU = _grouped_wgrad(gYg, t["act"], El, t["ts_l"], scale=inv_ep,
                                          passenger=(d_act, t["pre"], cfg.activation))
            else:
                d_act = ops.grouped_gemm(gYg, wd, _lib.B_NMAJOR, El, t["ts_l"], D, H)
                gU = ops.glu_backward(d_act, t["pre"], t["ts_l"], El, cfg.activation)
                d_wd = _grouped_wgrad(gYg, t["act"], El, t["ts_l"], scale=inv_ep)
            d_wu = _grouped_wgrad(gU, t["Xg"], El, t["ts_l"], scale=inv_ep)
            if cfg.ep_full_input_grad:
                # opt-in: the expert input gradient the reference leaves out (fused_moe.py:1001-1005) travels back
                # through a reverse dispatch exchange and is summed over each token's k slots
                dXg = ops.grouped_gemm(gU, wu, _lib.B_NMAJOR, El, t["ts_l"], 2 * H, D)
                dx_recv = dXg if direct else ops.combine_forward(dXg, t["pos_l"], None, M, 1)
                if has_latent:
                    dx_recv = ops.grouped_gemm(dx_recv, t["lwu"], _lib.B_NMAJOR, 1, None, D, L)
        else:
            d_wd = torch.zeros_like(wd)
            d_wu = torch.zeros_like(wu)
        if has_latent:
            # fused_moe.py:989-999: both un-projection sites feed proj_up, the combine projection feeds proj_down
            d_lwu = ops.grouped_gemm_wgrad(gYw, t["returned_lat"], 1, _dense_ts(T, h.device), scale=inv_ep)[0]
            if M > 0:
                ts_m = _dense_ts(recv_grad.shape[0], h.device)   # M rows, or the grouped rows with zero padding
                d_lwu = d_lwu + ops.grouped_gemm_wgrad(recv_grad, t["recv_lat"], 1, ts_m, scale=inv_ep)[0]
                d_lwd = ops.grouped_gemm_wgrad(recv_grad_lat, t["local_out_D"], 1, ts_m, scale=inv_ep)[0]
            else:
                d_lwd = torch.zeros_like(t["lwd"])

        if cfg.ep_full_input_grad:
            W = L if has_latent else D
            back = dx_recv if M > 0 else h.new_empty(0, W)
            if direct:
                d_send = plan.combine_grouped(back, 1)                             # [T, W], send order
            else:
                d_send, _ = plan.exchange(back, True, 1)
            d_disp = ops.combine_forward(d_send, t["cpos"], None, N, k)            # sum over the k slots
            if has_latent:
                d_disp = ops.grouped_gemm(d_disp, t["lwd"], _lib.B_NMAJOR, 1, None, L, D)
            dH = dH + d_disp
        s_grads = (None, None, None)
        if has_shared:
            torch.cuda.current_stream().wait_event(shared_done)
            dH = dH + s_dx
            s_grads = (s_dwg, s_dwu, s_dwd)
        dt = ctx.in_dtypes

        def cast(x, i):
            return None if x is None or dt[i] is None else x.to(dt[i])

        return (cast(dH, 0), cast(d_gate, 1), cast(d_wu, 2), cast(d_wd, 3), cast(s_grads[0], 4), cast(s_grads[1], 5),
                cast(s_grads[2], 6), cast(d_lwd, 7), cast(d_lwu, 8), None, None)


# ----------------------------------------------------------------------------------------------
# Public API
# ----------------------------------------------------------------------------------------------

@torch.compiler.disable
def set_ep_group(group, backend="nccl"):
    """Store the expert-parallel process group for later fused_moe() calls (reference: fused_moe.py:1026-1040)."""
    global _EP_GROUP, _EP_ACTIVE, _EP_BACKEND
    if group is not None and backend != "nccl":
        raise ValueError(f"ep backend {backend!r} is not available; use 'nccl'")
    _EP_GROUP = group
    _EP_ACTIVE = group is not None
    _EP_BACKEND = backend if group is not None else "nccl"


def _metrics(losses, counts, N, top_k, capacity_factor, E):
    tpe = counts.to(torch.float32)
    losses["tokens_per_expert"] = counts.to(torch.int32)
    losses["max_expert_load"] = tpe.max().int()
    losses["min_expert_load"] = tpe.min().int()
    losses["expert_load_imbalance"] = tpe.max() / (tpe.mean() + _WEIGHT_EPS)


@torch.compiler.disable
def fused_moe(
    hidden_states,            # [N, D]
    gate_weight,              # [E, D]
    w_up,                     # [E, ffn_dim, D]  (gate rows, then up rows)
    w_down,                   # [E, D, ffn_dim // 2]
    top_k=2,
    activation="swiglu",
    gating="softmax",
    capacity_factor=None,
    aux_loss_coeff=0.0,
    z_loss_coeff=0.0,
    recompute_activations=False,
    ep_group=None,
    max_tokens_per_expert=None,
    allow_dropped_tokens=False,
    return_metrics=False,
    shared_expert_weights=None,
    latent_weights=None,
    n_group=None,
    topk_group=None,
    scoring_factor=None,
    pre_softmax=False,
    input_jitter=0.0,
    expert_bias=None,
    ep_full_input_grad=False,
    _addend=None,
    _addend_ready=None,
    _shared=None,
):
    """Fused MoE forward; returns (output [N, D], losses dict). Arguments as in the reference
    (fused_moe.py:1073-1138). `_addend` is a private hook used by MoELayer to fold the shared expert's output
    into the combine kernel; `_shared` = (gate, up, down weights, activation) is the private hook with which MoELayer
    hands its shared expert to the single-GPU layer (the public `shared_expert_weights` keeps the reference's meaning:
    expert parallel only)."""
    group = ep_group if ep_group is not None else (_EP_GROUP if _EP_ACTIVE else None)
    if not _EP_ACTIVE:
        _validate_inputs(hidden_states, gate_weight, w_up, w_down, top_k, activation, gating, ep_group=ep_group)
    else:
        assert hidden_states.dim() == 2, f"hidden_states must be 2D [N, D], got {hidden_states.shape}"
        assert w_up.shape[0] < gate_weight.shape[0] or torch.distributed.get_world_size(group) == 1, \
            f"EP mode: w_up should have E_local < E experts, got {w_up.shape[0]} >= {gate_weight.shape[0]}"
        assert 1 <= top_k <= gate_weight.shape[0], f"top_k must be in [1, {gate_weight.shape[0]}], got {top_k}"
        assert activation in ("swiglu", "geglu", "relu_squared"), f"Unknown activation: {activation}"
        assert gating in ("softmax", "sigmoid"), f"Unknown gating: {gating}"
    if not hidden_states.is_cuda:
        raise RuntimeError("flashfusedmoe_b200 runs on CUDA (sm_100a) tensors only; there is no CPU path")

    N, D = hidden_states.shape
    E = gate_weight.shape[0]
    dtype = _require_bf16(_get_compute_dtype(hidden_states.dtype))
    use_groups = n_group is not None and topk_group is not None
    if use_groups:
        assert E % n_group == 0, f"E ({E}) must be divisible by n_group ({n_group})"
    capacity = None
    if capacity_factor is not None and group is None:
        capacity = max(int((N / E) * capacity_factor), top_k)  # fused_moe.py:352-353
    cfg = _Cfg(top_k=top_k, activation=activation, gating=gating, aux_loss_coeff=float(aux_loss_coeff),
               z_loss_coeff=float(z_loss_coeff), recompute=bool(recompute_activations), expert_bias=expert_bias,
               weight_scale=1.0 if scoring_factor is None else float(scoring_factor) / top_k,
               aux_grad=_AUX_LOSS_GRAD, ep_group=group, ep_full_input_grad=bool(ep_full_input_grad),
               pre_softmax=bool(pre_softmax) and gating == "softmax", n_group=int(n_group) if use_groups else 0,
               topk_group=int(topk_group) if use_groups else 0, capacity=capacity,
               input_jitter=float(input_jitter or 0.0), addend_ready=_addend_ready)
    sw_all = shared_expert_weights if shared_expert_weights is not None else ()
    lw_all = latent_weights if latent_weights is not None else ()
    cfg.wants_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad
        for t in (hidden_states, gate_weight, w_up, w_down, _addend, *sw_all, *lw_all,
                  *(_shared[:3] if _shared is not None else ())))

    if group is not None:
        sw = shared_expert_weights if shared_expert_weights is not None else (None, None, None)
        lw = latent_weights if latent_weights is not None else (None, None)
        if (_EP_STATIC_TOKENS is not None and lw[0] is None and _EP_TRANSPORT == "p2p" and p2p.available()
                and E % 4 == 0 and E <= 256 and torch.distributed.get_world_size(group) <= 16):
            out, aux, z, counts, dropped = _FusedMoEEPStaticFunction.apply(hidden_states, gate_weight, w_up, w_down,
                                                                           sw[0], sw[1], sw[2], cfg, dtype)
        else:
            out, aux, z, counts, dropped = _FusedMoEEPFunction.apply(hidden_states, gate_weight, w_up, w_down, sw[0],
                                                                     sw[1], sw[2], lw[0], lw[1], cfg, dtype)
    else:
        sh = (None, None, None)
        if _shared is not None:
            sh = tuple(_shared[:3])
            cfg.shared_activation = _shared[3]
        out, aux, z, counts, dropped = _FusedMoEFunction.apply(hidden_states, gate_weight, w_up, w_down, _addend,
                                                               sh[0], sh[1], sh[2], cfg, dtype)
        if max_tokens_per_expert is not None and not allow_dropped_tokens and capacity is None:
            actual_max = int(counts.max().item())
            if actual_max > max_tokens_per_expert:
                raise RuntimeError(
                    f"MoE routing overflow: expert received {actual_max} tokens but buffer "
                    f"is {max_tokens_per_expert}. {actual_max - max_tokens_per_expert} tokens exceed the bound "
                    f"given by max_tokens_per_expert. Fix options:\n"
                    f"  1. Set max_tokens_per_expert={actual_max} (or higher) via calibration\n"
                    f"  2. Set allow_dropped_tokens=True to suppress this error")

    # a device-side failure of an earlier call (bounded wait that ran out, bad index) raises here; no GPU wait
    ops.poll_status(hidden_states.device)

    losses = {}
    if aux_loss_coeff > 0.0:
        losses["aux_loss"] = aux
    if z_loss_coeff > 0.0:
        losses["z_loss"] = z
    if return_metrics:
        _metrics(losses, counts, N, top_k, capacity_factor, E)
        if capacity_factor is not None:
            losses["dropped_token_count"] = dropped.reshape(()).to(torch.int64)
            losses["dropped_token_fraction"] = dropped.reshape(()).float() / (N * top_k)
    return out, losses
