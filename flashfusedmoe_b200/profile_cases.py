"""One kernel at the single-GPU benchmark shape, a few launches, for `ncu` captures and quick timing.

    python -m flashfusedmoe_b200.profile_cases <case> [--launches 3] [--experts 8] [--rows-per-expert 4096]

Cases: route_forward permute combine_forward combine_backward glu_backward route_backward
       gemm_up_glu gemm_down gemm_dact gemm_dx gemm_wgrad_down gemm_wgrad_up
       quantize_rows gemm_up_glu_fp8 gemm_down_fp8 gemm_dact_glu_bwd
Shape: D = 1024, H = 2048, top_k = 2 (E * rows_per_expert routed rows). Every case touches far more than the
126 MB L2 and holds about 1 GB on the device. Prints the CUDA-event time per launch.
"""

import argparse

import torch

from . import _lib, ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--rows-per-expert", type=int, default=4096)
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--half-ffn", type=int, default=2048)
    a = ap.parse_args()
    dev = "cuda"
    torch.manual_seed(0)
    E, D, H, k = a.experts, a.d_model, a.half_ffn, 2
    T = E * a.rows_per_expert
    N = T // k
    ts = torch.arange(E + 1, dtype=torch.int32, device=dev) * (a.rows_per_expert // 128)
    hidden = torch.randn(N, D, device=dev).bfloat16()
    gate = (torch.randn(E, D, device=dev) * 0.02).bfloat16()
    r = ops.route_forward(hidden, gate, k, "softmax")
    rows = r.rows_cap
    X = torch.randn(rows, D, device=dev).bfloat16()
    Wu = (torch.randn(E, 2 * H, D, device=dev) * 0.02).bfloat16()
    Wd = (torch.randn(E, D, H, device=dev) * 0.02).bfloat16()
    act = torch.randn(rows, H, device=dev).bfloat16()
    pre = torch.randn(rows, 2 * H, device=dev).bfloat16()
    gU = torch.randn(rows, 2 * H, device=dev).bfloat16()
    gw = torch.randn(N * k, device=dev)
    cases = {
        "route_forward": (lambda: ops.route_forward(hidden, gate, k, "softmax"), None),
        "permute": (lambda: ops.permute_rows(hidden, r.src, rows, k), 2.0 * T * D * 2),
        "combine_forward": (lambda: ops.combine_forward(X, r.pos, r.topk_w, N, k), (T + N) * D * 2.0),
        "combine_backward": (lambda: ops.combine_backward(hidden, X, r.topk_w, r.src, rows, k), (2 * T + N) * D * 2.0),
        "glu_backward": (lambda: ops.glu_backward(act, pre, r.tile_start, E, "swiglu"), 5.0 * T * H * 2),
        "route_backward": (lambda: ops.route_backward(gw, r, None, None, hidden, gate, "softmax"), None),
        "gemm_up_glu": (lambda: ops.grouped_gemm_glu(X, Wu, Wu.view(-1, D)[H:], 2 * H, E, ts, D, H, "swiglu"),
                        4.0 * T * D * H),
        "gemm_down": (lambda: ops.grouped_gemm(act, Wd, _lib.B_KMAJOR, E, ts, H, D), 2.0 * T * D * H),
        "gemm_dact": (lambda: ops.grouped_gemm(X, Wd, _lib.B_NMAJOR, E, ts, D, H), 2.0 * T * D * H),
        "gemm_dact_glu_bwd": (lambda: ops.grouped_gemm_dact_glu_backward(X, Wd, E, ts, D, H, pre, "swiglu"),
                              2.0 * T * D * H),
        "gemm_dx": (lambda: ops.grouped_gemm(gU, Wu, _lib.B_NMAJOR, E, ts, 2 * H, D), 4.0 * T * D * H),
        "gemm_wgrad_down": (lambda: ops.grouped_gemm_wgrad(X, act, E, ts), 2.0 * T * D * H),
        "gemm_wgrad_up": (lambda: ops.grouped_gemm_wgrad(gU, X, E, ts), 4.0 * T * D * H),
    }
    if a.case in ("quantize_rows", "gemm_up_glu_fp8", "gemm_down_fp8"):
        xq, xs = ops.quantize_rows_e4m3(X)
        wuq, wus = ops.quantize_weight_e4m3(Wu)
        aq, as_ = ops.quantize_rows_e4m3(act)
        wdq, wds = ops.quantize_weight_e4m3(Wd)
        cases.update({
            "quantize_rows": (lambda: ops.quantize_rows_e4m3(act), 3.0 * rows * H),
            "gemm_up_glu_fp8": (lambda: ops.grouped_gemm_glu_fp8(xq, xs, wuq, wus, E, ts, D, H, "swiglu"),
                                4.0 * T * D * H),
            "gemm_down_fp8": (lambda: ops.grouped_gemm_fp8(aq, as_, wdq, wds, E, ts, H, D), 2.0 * T * D * H),
        })
    fn, work = cases[a.case]
    fn()
    torch.cuda.synchronize()
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.launches):
        fn()
    e.record()
    torch.cuda.synchronize()
    ops.check_status()
    ms = s.elapsed_time(e) / a.launches
    unit = ""
    if work is not None:
        unit = f"  {work / ms / 1e9:.1f} {'TFLOP/s' if a.case.startswith('gemm') else 'GB/s (x1e-3: TB/s)'}"
        if not a.case.startswith("gemm"):
            unit = f"  {work / ms / 1e6:.1f} GB/s"
    print(f"{a.case}: {ms:.4f} ms per launch{unit}")


if __name__ == "__main__":
    main()
