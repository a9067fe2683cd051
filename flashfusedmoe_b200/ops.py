"""Tensor-level wrappers around the libffmoe C ABI.

Each function takes CUDA bf16/int32/float32 tensors, allocates outputs through torch's caching allocator
and enqueues the kernels on the current CUDA stream. Nothing here computes on the host; without a GPU
or without the built library every call raises.
"""

from dataclasses import dataclass

import torch

from . import _lib

_status = {}
_workspaces = {}

# Instrumentation used by bench.py: a launch counter (kernels of this library enqueued so far) and an
# optional per-kernel CUDA-event timer on the launching stream.
launch_count = 0
a2a_bytes_sent = 0
_timer = None


class KernelTimer:
    """Records a CUDA-event pair around selected kernel launches while installed with set_timer()."""

    def __init__(self):
        self.events = {}

    def totals_ms(self):
        """name -> (launches, total milliseconds); call after torch.cuda.synchronize()."""
        return {n: (len(ev), sum(a.elapsed_time(b) for a, b in ev)) for n, ev in self.events.items()}

    def union_ms(self, names, exclude=()):
        """Milliseconds during which at least one launch filed under `names` (and not under `exclude`) was between its
        start and its end event. Launches on different streams overlap in time: a kernel whose start event has fired
        may still wait for the SMs that a kernel of another stream holds, so the sum of the event pairs counts that
        time twice and the merged intervals count it once. Call after torch.cuda.synchronize()."""
        skip = {id(p) for n in exclude for p in self.events.get(n, ())}
        pairs = {id(p): p for n in names for p in self.events.get(n, ()) if id(p) not in skip}
        if not pairs:
            return 0.0
        base = next(iter(pairs.values()))[0]
        spans = sorted((base.elapsed_time(a), base.elapsed_time(b)) for a, b in pairs.values())
        total, lo, hi = 0.0, spans[0][0], spans[0][1]
        for a, b in spans[1:]:
            if a > hi:
                total += hi - lo
                lo, hi = a, b
            else:
                hi = max(hi, b)
        return total + (hi - lo)


def set_timer(timer):
    global _timer
    _timer = timer


class _Launch:
    """Counts `kernels` launches under `name`; with a timer installed also brackets them with events."""

    def __init__(self, name, kernels=1, also=None):
        self.name = name
        self.kernels = kernels
        self.also = also   # second timer bucket for the same event pair (a finer breakdown of `name`)

    def __enter__(self):
        global launch_count
        launch_count += self.kernels
        if _timer is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if _timer is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            _timer.events.setdefault(self.name, []).append((self.start, end))
            if self.also is not None:
                _timer.events.setdefault(self.also, []).append((self.start, end))
        return False


def _ptr(t):
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """cudaStream_t of torch's current stream on the current device (the raw getter avoids building a Stream object:
    this is called once per kernel launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _req(t, dtype, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: flashfusedmoe_b200 has no CPU path")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def status_tensor(device):
    """Per-device int32 status word written by kernels whose bounded waits ran out."""
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status[key]


def check_status(device=None):
    """Synchronise and raise if any kernel reported a device-side failure since the last check."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = status_tensor(dev)
    code = int(st.item())
    # an asynchronous copy of the word queued by poll_status() carries the same information: drop it, so that a failure
    # reported here is not reported a second time by a later fused_moe() call
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    entry = _status_host.get(key)
    if entry is not None and entry["pending"]:
        entry["done"].synchronize()
        entry["pending"] = False
        entry["host"][0] = 0
    if code != 0:
        st.zero_()
        raise RuntimeError(f"libffmoe device status {code}: {_lib.error_string(code)}")


_status_host = {}


def poll_status(device=None, enqueue=True):
    """Host-side check of the status word that never waits for the GPU.

    The word is copied to pinned host memory asynchronously (a 4-byte copy on a stream of its own, ordered after
    the work queued so far, so the compute streams never wait for it); once that copy has finished its value is
    read here and a non-zero code raises, so a bounded wait that ran out inside one call surfaces at a later call
    instead of as silent garbage. With `enqueue` a fresh copy is queued for the next poll. Does nothing while the
    current stream is being captured into a CUDA graph."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if torch.cuda.is_current_stream_capturing():
        return
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    entry = _status_host.get(key)
    if entry is None:
        entry = _status_host[key] = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "pending": False,
                                     "stream": torch.cuda.Stream(device=dev), "ready": torch.cuda.Event(),
                                     "done": torch.cuda.Event()}
    if entry["pending"]:
        if not entry["done"].query():
            return  # the last copy is still in flight: look again at the next call
        entry["pending"] = False
        code = int(entry["host"][0])
        if code != 0:
            entry["host"][0] = 0
            status_tensor(dev).zero_()
            raise RuntimeError(f"libffmoe device status {code}: {_lib.error_string(code)} "
                               "(reported by a kernel of an earlier call; its results are not valid)")
    if enqueue:
        side = entry["stream"]
        entry["ready"].record()
        side.wait_event(entry["ready"])
        with torch.cuda.stream(side):
            entry["host"].copy_(status_tensor(dev), non_blocking=True)
            entry["done"].record(side)
        entry["pending"] = True


def raise_on_status(code, device):
    """Raise for a status code the caller already holds on the host (read together with other data)."""
    code = int(code)
    if code != 0:
        status_tensor(device).zero_()
        raise RuntimeError(f"libffmoe device status {code}: {_lib.error_string(code)}")


def rows_capacity(T, E):
    return int(_lib.load().ffm_rows_capacity(int(T), int(E)))


def _workspace(device, nbytes, tag):
    """Grow-only scratch buffer per (device, tag); reused across calls on the same stream order."""
    key = (torch.device(device).index, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


@dataclass
class Routing:
    """Everything the routing kernels produce for one call (see include/ffmoe.h for the layout)."""
    topk_w: torch.Tensor      # [N, k] f32
    topk_idx: torch.Tensor    # [N, k] int32
    logits: torch.Tensor      # [N, E] bf16
    lse: torch.Tensor         # [N] f32
    counts: torch.Tensor      # [E] int32
    tile_start: torch.Tensor  # [E + 1] int32
    pos: torch.Tensor         # [N * k] int32
    src: torch.Tensor         # [rows_cap] int32
    stats: torch.Tensor       # [E + 2] f32
    rows_cap: int
    top_k: int
    num_experts: int


def route_forward(hidden, gate_w, top_k, gating="softmax", expert_bias=None, weight_scale=1.0, pre_softmax=False,
                  n_group=0, topk_group=0):
    lib = _lib.load()
    _req(hidden, torch.bfloat16, "hidden")
    _req(gate_w, torch.bfloat16, "gate_w")
    N, D = hidden.shape
    E = gate_w.shape[0]
    dev = hidden.device
    T = N * top_k
    rows_cap = rows_capacity(T, E)
    if expert_bias is not None:
        expert_bias = _req(expert_bias.to(torch.float32).contiguous(), torch.float32, "expert_bias")
    r = Routing(
        topk_w=torch.empty(N, top_k, dtype=torch.float32, device=dev),
        topk_idx=torch.empty(N, top_k, dtype=torch.int32, device=dev),
        logits=torch.empty(N, E, dtype=torch.bfloat16, device=dev),
        lse=torch.empty(N, dtype=torch.float32, device=dev),
        counts=torch.empty(E, dtype=torch.int32, device=dev),
        tile_start=torch.empty(E + 1, dtype=torch.int32, device=dev),
        pos=torch.empty(T, dtype=torch.int32, device=dev),
        src=torch.empty(max(rows_cap, 1), dtype=torch.int32, device=dev),
        stats=torch.empty(E + 2, dtype=torch.float32, device=dev),
        rows_cap=rows_cap, top_k=top_k, num_experts=E)
    ws_bytes = int(lib.ffm_route_workspace_bytes(N, E, top_k))
    ws = _workspace(dev, ws_bytes, "route")
    with _Launch("route_forward", 3):
        rc = lib.ffm_route_forward(_ptr(hidden), _ptr(gate_w), _ptr(expert_bias), N, D, E, top_k,
                                   _lib.GATING[gating], float(weight_scale), 1 if pre_softmax else 0, int(n_group or 0),
                                   int(topk_group or 0), _ptr(r.logits), _ptr(r.topk_w),
                                   _ptr(r.topk_idx), _ptr(r.lse), _ptr(r.counts), _ptr(r.tile_start), _ptr(r.pos),
                                   _ptr(r.src), rows_cap, _ptr(r.stats), _ptr(ws), ws.numel(),
                                   _ptr(status_tensor(dev)), _stream())
    _lib.check(rc, "ffm_route_forward")
    return r


def route_apply_capacity(r, capacity):
    """Drop slots beyond `capacity` per expert in place (weights renormalised, rows turned into padding).
    Returns the int32 [1] count of dropped slots."""
    lib = _lib.load()
    dropped = torch.empty(1, dtype=torch.int32, device=r.topk_w.device)
    N = r.topk_w.shape[0]
    with _Launch("route_capacity", 1):
        rc = lib.ffm_route_apply_capacity(_ptr(r.topk_w), _ptr(r.topk_idx), _ptr(r.pos), _ptr(r.src),
                                          _ptr(r.tile_start), N, r.top_k, r.num_experts, int(capacity), _ptr(dropped),
                                          _stream())
    _lib.check(rc, "ffm_route_apply_capacity")
    return dropped


def group_rows(expert_ids, num_experts):
    """Grouped-row map for rows already tagged with an expert id (int32 [T])."""
    lib = _lib.load()
    _req(expert_ids, torch.int32, "expert_ids")
    T = expert_ids.numel()
    dev = expert_ids.device
    rows_cap = rows_capacity(T, num_experts)
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    tile_start = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    pos = torch.empty(max(T, 1), dtype=torch.int32, device=dev)
    src = torch.empty(max(rows_cap, 1), dtype=torch.int32, device=dev)
    ws_bytes = int(lib.ffm_route_workspace_bytes(max(T, 1), num_experts, 1))
    ws = _workspace(dev, ws_bytes, "group")
    with _Launch("group_rows", 3):
        rc = lib.ffm_group_rows(_ptr(expert_ids), T, num_experts, _ptr(counts), _ptr(tile_start), _ptr(pos), _ptr(src),
                                rows_cap, _ptr(ws), ws.numel(), _ptr(status_tensor(dev)), _stream())
    _lib.check(rc, "ffm_group_rows")
    return counts, tile_start, pos[:T], src, rows_cap


def permute_rows(x, src, rows_cap, top_k, zero_padding=True):
    """grouped[r] = x[src[r] // top_k]; padding rows (src < 0) are zeroed unless zero_padding is False."""
    lib = _lib.load()
    _req(x, torch.bfloat16, "x")
    _req(src, torch.int32, "src")
    D = x.shape[1]
    out = torch.empty(rows_cap, D, dtype=torch.bfloat16, device=x.device)
    with _Launch("permute_rows", 1):
        _lib.check(lib.ffm_permute_rows(_ptr(x), _ptr(src), rows_cap, top_k, D, 1 if zero_padding else 0, _ptr(out),
                                        _stream()), "ffm_permute_rows")
    return out


def compact_positions(routing, T):
    """(cpos, src_c): send-order position of every flat slot and its inverse (ffm_compact_positions)."""
    lib = _lib.load()
    dev = routing.pos.device
    cpos = torch.empty(T, dtype=torch.int32, device=dev)
    src_c = torch.empty(T, dtype=torch.int32, device=dev)
    with _Launch("compact_positions", 1):
        rc = lib.ffm_compact_positions(_ptr(routing.pos), _ptr(routing.topk_idx), _ptr(routing.counts),
                                       _ptr(routing.tile_start), T, routing.counts.numel(), _ptr(cpos), _ptr(src_c),
                                       _stream())
    _lib.check(rc, "ffm_compact_positions")
    return cpos, src_c


def grouped_gemm_glu(A, w_gate, w_up, group_rows_, groups, tile_start, K, H, activation, want_preact=True,
                     valid_rows=None, tile_rows=0):
    """act = glu(A Wg^T, A Wu^T). w_gate / w_up are tensors whose data pointers address the first gate / up row.
    valid_rows (int32 [groups], device): tiles beyond a group's valid rows are skipped; tile_rows 128 / 256 picks the
    tile shape for this call (0 = library default)."""
    lib = _lib.load()
    _req(A, torch.bfloat16, "A")
    rows = A.shape[0]
    act = torch.empty(rows, H, dtype=torch.bfloat16, device=A.device)
    pre = torch.empty(rows, 2 * H, dtype=torch.bfloat16, device=A.device) if want_preact else None
    with _Launch("gemm_up_glu", 1):
        rc = lib.ffm_grouped_gemm_glu(_ptr(A), _ptr(w_gate), _ptr(w_up), group_rows_, groups, _ptr(tile_start), rows, K,
                                      H, _lib.ACTIVATION[activation], _ptr(act), _ptr(pre), _ptr(valid_rows),
                                      int(tile_rows), _ptr(status_tensor(A.device)), _stream())
    _lib.check(rc, "ffm_grouped_gemm_glu")
    return act, pre


def grouped_gemm(A, B, b_major, groups, tile_start, K, n_out, scale=1.0, valid_rows=None, tile_rows=0):
    lib = _lib.load()
    _req(A, torch.bfloat16, "A")
    _req(B, torch.bfloat16, "B")
    rows = A.shape[0]
    out = torch.empty(rows, n_out, dtype=torch.bfloat16, device=A.device)
    with _Launch("gemm", 1):
        rc = lib.ffm_grouped_gemm(_ptr(A), _ptr(B), b_major, groups, _ptr(tile_start), rows, K, n_out, float(scale),
                                  _ptr(out), _ptr(valid_rows), int(tile_rows), _ptr(status_tensor(A.device)),
                                  _stream())
    _lib.check(rc, "ffm_grouped_gemm")
    return out


def grouped_gemm_wgrad(A, B, groups, tile_start, scale=1.0):
    """dW[e] = scale * A[rows of e]^T B[rows of e]; A [rows_cap, M], B [rows_cap, N] -> [groups, M, N]."""
    lib = _lib.load()
    _req(A, torch.bfloat16, "A")
    _req(B, torch.bfloat16, "B")
    rows_cap, M = A.shape
    n_out = B.shape[1]
    out = torch.empty(groups, M, n_out, dtype=torch.bfloat16, device=A.device)
    with _Launch("gemm_wgrad", 1):
        rc = lib.ffm_grouped_gemm_wgrad(_ptr(A), _ptr(B), groups, _ptr(tile_start), rows_cap, M, n_out, float(scale),
                                        _ptr(out), _ptr(status_tensor(A.device)), _stream())
    _lib.check(rc, "ffm_grouped_gemm_wgrad")
    return out


def grouped_gemm_wgrad_glu_backward(A, B, groups, tile_start, d_act, preact, activation, scale=1.0):
    """(dW, gU): grouped_gemm_wgrad(A, B) and glu_backward(d_act, preact) in one launch, the second riding on extra
    warps of the GEMM's CTAs (ffm_grouped_gemm_wgrad_glu_backward). Bit-identical to the two separate calls; rows past
    the last group's tiles are left untouched."""
    lib = _lib.load()
    _req(A, torch.bfloat16, "A")
    _req(B, torch.bfloat16, "B")
    _req(d_act, torch.bfloat16, "d_act")
    _req(preact, torch.bfloat16, "preact")
    rows_cap, M = A.shape
    n_out = B.shape[1]
    rows, H = d_act.shape
    out = torch.empty(groups, M, n_out, dtype=torch.bfloat16, device=A.device)
    gU = torch.empty(rows, 2 * H, dtype=torch.bfloat16, device=A.device)
    with _Launch("gemm_wgrad", 1, also="gemm_wgrad_passenger"):
        rc = lib.ffm_grouped_gemm_wgrad_glu_backward(_ptr(A), _ptr(B), groups, _ptr(tile_start), rows_cap, M, n_out,
                                                     float(scale), _ptr(out), _ptr(d_act), _ptr(preact), rows, H,
                                                     _lib.ACTIVATION[activation], _ptr(gU),
                                                     _ptr(status_tensor(A.device)), _stream())
    _lib.check(rc, "ffm_grouped_gemm_wgrad_glu_backward")
    return out, gU


def grouped_gemm_dact_glu_backward(gY, Wd, groups, tile_start, K, H, preact, activation):
    """gU [rows, 2H]: the dAct GEMM (gY Wd, N-major B) with the GLU backward in its epilogue; equals
    glu_backward(grouped_gemm(gY, Wd, B_NMAJOR, ...), preact) bit for bit without writing dAct."""
    lib = _lib.load()
    _req(gY, torch.bfloat16, "gY")
    _req(Wd, torch.bfloat16, "Wd")
    _req(preact, torch.bfloat16, "preact")
    rows = gY.shape[0]
    gU = torch.empty(rows, 2 * H, dtype=torch.bfloat16, device=gY.device)
    with _Launch("gemm", 1, also="gemm_dact_glu_backward"):
        rc = lib.ffm_grouped_gemm_dact_glu_backward(_ptr(gY), _ptr(Wd), groups, _ptr(tile_start), rows, K, H,
                                                    _lib.ACTIVATION[activation], _ptr(preact), _ptr(gU), 0,
                                                    _ptr(status_tensor(gY.device)), _stream())
    _lib.check(rc, "ffm_grouped_gemm_dact_glu_backward")
    return gU


def quantize_rows_e4m3(x):
    """(q uint8 [rows, K], scale f32 [rows padded to 128]): row-wise e4m3 quantisation, x = q * scale[row]."""
    lib = _lib.load()
    _req(x, torch.bfloat16, "x")
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=torch.uint8, device=x.device)
    scale = torch.ones((rows + 127) // 128 * 128, dtype=torch.float32, device=x.device)
    with _Launch("quantize_rows", 1):
        _lib.check(lib.ffm_quantize_rows_e4m3(_ptr(x), rows, K, _ptr(q), _ptr(scale), _stream()),
                   "ffm_quantize_rows_e4m3")
    return q, scale


def quantize_weight_e4m3(w):
    """(q uint8 [E, N, K], scale f32 [E]): e4m3 copy of a weight tensor with one scale per expert,
    w[e] = q[e] * scale[e]. Two launches: per-row maxima, then the conversion with the per-expert scale."""
    lib = _lib.load()
    _req(w, torch.bfloat16, "w")
    E, N, K = w.shape
    flat = w.reshape(E * N, K)
    _, row_scale = quantize_rows_e4m3(flat)
    scale = row_scale[:E * N].view(E, N).amax(dim=1).contiguous()
    q = torch.empty(E, N, K, dtype=torch.uint8, device=w.device)
    with _Launch("quantize_rows", 1):
        _lib.check(lib.ffm_quantize_rows_given_scale_e4m3(_ptr(flat), E * N, K, N, _ptr(scale), _ptr(q), _stream()),
                   "ffm_quantize_rows_given_scale_e4m3")
    return q, scale


def grouped_gemm_glu_fp8(Aq, a_scale, Wq, w_scale, groups, tile_start, K, H, activation, want_preact=True,
                         tile_rows=0):
    """grouped_gemm_glu on e4m3 operands: Aq uint8 [rows, K] with a scale per row (quantize_rows_e4m3), Wq uint8
    [groups, 2H, K] with a scale per group (quantize_weight_e4m3). Outputs bf16."""
    lib = _lib.load()
    rows = Aq.shape[0]
    act = torch.empty(rows, H, dtype=torch.bfloat16, device=Aq.device)
    pre = torch.empty(rows, 2 * H, dtype=torch.bfloat16, device=Aq.device) if want_preact else None
    with _Launch("gemm_up_glu", 1):
        rc = lib.ffm_grouped_gemm_glu_fp8(_ptr(Aq), _ptr(a_scale), _ptr(Wq), _ptr(w_scale), groups, _ptr(tile_start),
                                          rows, K, H, _lib.ACTIVATION[activation], _ptr(act), _ptr(pre),
                                          int(tile_rows), _ptr(status_tensor(Aq.device)), _stream())
    _lib.check(rc, "ffm_grouped_gemm_glu_fp8")
    return act, pre


def grouped_gemm_fp8(Aq, a_scale, Bq, b_scale, groups, tile_start, K, n_out, tile_rows=0):
    """grouped_gemm (K-major B) on e4m3 operands: Bq uint8 [groups, n_out, K]. Output bf16 [rows, n_out]."""
    lib = _lib.load()
    rows = Aq.shape[0]
    out = torch.empty(rows, n_out, dtype=torch.bfloat16, device=Aq.device)
    with _Launch("gemm", 1):
        rc = lib.ffm_grouped_gemm_fp8(_ptr(Aq), _ptr(a_scale), _ptr(Bq), _ptr(b_scale), groups, _ptr(tile_start), rows,
                                      K, n_out, _ptr(out), int(tile_rows), _ptr(status_tensor(Aq.device)), _stream())
    _lib.check(rc, "ffm_grouped_gemm_fp8")
    return out


def combine_forward(Y, pos, w, N, top_k, addend=None):
    lib = _lib.load()
    _req(Y, torch.bfloat16, "Y")
    _req(pos, torch.int32, "pos")
    D = Y.shape[1]
    out = torch.empty(N, D, dtype=torch.bfloat16, device=Y.device)
    with _Launch("combine_forward", 1):
        rc = lib.ffm_combine_forward(_ptr(Y), _ptr(pos), _ptr(w), _ptr(addend), N, top_k, D, _ptr(out), _stream())
    _lib.check(rc, "ffm_combine_forward")
    return out


def combine_backward(go, Y, w, src, rows_cap, top_k, want_gw=True):
    lib = _lib.load()
    _req(go, torch.bfloat16, "go")
    D = go.shape[1]
    gYw = torch.empty(rows_cap, D, dtype=torch.bfloat16, device=go.device)
    gw = torch.zeros(go.shape[0] * top_k, dtype=torch.float32, device=go.device) if want_gw else None
    with _Launch("combine_backward", 1):
        rc = lib.ffm_combine_backward(_ptr(go), _ptr(Y if want_gw else None), _ptr(w), _ptr(src), rows_cap, top_k, D,
                                      _ptr(gYw), _ptr(gw), _stream())
    _lib.check(rc, "ffm_combine_backward")
    return gYw, gw


def glu_backward(dAct, preact, tile_start, groups, activation):
    lib = _lib.load()
    _req(dAct, torch.bfloat16, "dAct")
    _req(preact, torch.bfloat16, "preact")
    rows, H = dAct.shape
    gU = torch.empty(rows, 2 * H, dtype=torch.bfloat16, device=dAct.device)
    with _Launch("glu_backward", 1):
        rc = lib.ffm_glu_backward(_ptr(dAct), _ptr(preact), _ptr(tile_start), groups, rows, H,
                                  _lib.ACTIVATION[activation], _ptr(gU), _stream())
    _lib.check(rc, "ffm_glu_backward")
    return gU


def route_backward(gw, routing, gaux, gz, hidden, gate_w, gating, dH=None):
    """Returns (dH, dGate). If dH is given the routing term is added to it in place.
    gaux: f32 [E] device tensor or None; gz: f32 device scalar tensor or None."""
    lib = _lib.load()
    N, D = hidden.shape
    E = gate_w.shape[0]
    dev = hidden.device
    accumulate = dH is not None
    if dH is None:
        dH = torch.empty(N, D, dtype=torch.bfloat16, device=dev)
    dGate = torch.empty(E, D, dtype=torch.bfloat16, device=dev)
    ws_bytes = int(lib.ffm_route_backward_workspace_bytes(N, D, E))
    ws = _workspace(dev, ws_bytes, "route_bwd")
    with _Launch("route_backward", 3):
        rc = lib.ffm_route_backward(_ptr(gw), _ptr(routing.topk_w), _ptr(routing.topk_idx), _ptr(routing.logits),
                                    _ptr(routing.lse), _ptr(gaux), _ptr(gz), _ptr(hidden), _ptr(gate_w), N, D, E,
                                    routing.top_k, _lib.GATING[gating], 1 if accumulate else 0, _ptr(dH), _ptr(dGate),
                                    _ptr(ws), ws.numel(), _ptr(status_tensor(dev)), _stream())
    _lib.check(rc, "ffm_route_backward")
    return dH, dGate
