"""The unmodified reference on the GPU beside this package, same process, same weights, same tokens.

Test and measurement infrastructure (like everything under oracle/): never imported by the product.

    python -m pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <reference checkout>
    python oracle/reference_on_gpu.py [--steps 20] [--warmup 8] [--config 2|3|5]

Imports `flashfusemoe` (the reference, installed unmodified into the git-ignored baseline/_ref) and runs its own
`MoELayer` at BASELINE configs[1] on cuda:0: bf16, seed 1, weights N(0, 0.02), x [8, 2048, 1024], one shared
expert, forward + backward with an explicit dense grad_output. `max_tokens_per_expert` is set to the largest
per-expert count of this input so that the reference's padded [E, max_tokens, D] buffer drops nothing (its
default bound is an estimate and rows beyond it are silently mis-routed). This package's MoELayer loads the
reference layer's state dict (strict) and runs the same step. Both are timed with CUDA events after warm-up
(the reference's Triton kernels autotune during it), K steps in one bracket, and compared:
outputs, every gradient (max |a - b| / max |b|) and the per-expert token counts.
`--config 3` (BASELINE configs[2], Mixtral-shaped, fp32 Zipf(1.1) `expert_bias`, forward + backward) and `--config 5`
(BASELINE configs[4], decode shape, 128 tokens, forward only under no_grad) call both packages' `fused_moe()`
directly on the same tensors.
Prints one JSON line. Needs Triton on the box; says so and exits 0 if the reference cannot be imported.
"""

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

import torch  # noqa: E402


def rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def timed(step, steps, warmup):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def functional_case(a, ref, ffm, ops):
    """configs[2] / configs[4] through fused_moe() of both packages on the same tensors."""
    dev = torch.device("cuda", 0)
    if a.config == 3:
        N, D, F, E, k, seed, train = 8192, 4096, 28672, 8, 2, 2, True
        name = "BASELINE configs[2]: D=4096 E=8 top_k=2 swiglu ffn_dim=2x14336, 8192 tokens, Zipf(1.1) gate bias, fwd+bwd"
    else:
        N, D, F, E, k, seed, train = 128, 7168, 4096, 256, 8, 4, False
        name = "BASELINE configs[4]: D=7168 E=256 top_k=8 swiglu ffn_dim=2x2048, 128 tokens, forward only"
    torch.manual_seed(seed)
    g = (torch.randn(E, D, device=dev) * 0.02).bfloat16()
    wu = (torch.randn(E, F, D, device=dev) * 0.02).bfloat16()
    wd = (torch.randn(E, D, F // 2, device=dev) * 0.02).bfloat16()
    x = torch.randn(N, D, device=dev).bfloat16()
    go = torch.randn(N, D, device=dev).bfloat16()
    bias = None
    if a.config == 3:
        gen = torch.Generator().manual_seed(seed)
        perm = torch.randperm(E, generator=gen)
        p = 1.0 / torch.arange(1, E + 1).float() ** 1.1
        bias = torch.log(p / p.sum())[perm].to(dev)
    with torch.no_grad():
        _, m = ffm.fused_moe(x, g, wu, wd, top_k=k, expert_bias=bias, return_metrics=True)
    tight = int(m["max_expert_load"])

    def make_step(fn, extra):
        ps = [t.clone().requires_grad_(train) for t in (x, g, wu, wd)]

        def step():
            if train:
                for t in ps:
                    t.grad = None
                out, _ = fn(*ps, top_k=k, expert_bias=bias, **extra)
                out.backward(go)
            else:
                with torch.no_grad():
                    out, _ = fn(*ps, top_k=k, expert_bias=bias, **extra)
            return out
        return step, ps

    r_step, r_ps = make_step(ref.fused_moe, dict(max_tokens_per_expert=tight, allow_dropped_tokens=True))
    o_step, o_ps = make_step(ffm.fused_moe, {})
    r_ms = min(timed(r_step, a.steps, a.warmup), timed(r_step, a.steps, 2))
    o_ms = min(timed(o_step, a.steps, a.warmup), timed(o_step, a.steps, 2))
    ops.check_status()
    out_r, out_o = r_step(), o_step()
    torch.cuda.synchronize()
    errs = {"out": rel(out_o, out_r)}
    if train:
        for n, a_, b_ in zip(("dH", "dGate", "dW_up", "dW_down"), o_ps, r_ps):
            errs[n] = rel(a_.grad, b_.grad)
    print(json.dumps({"workload": name, "gpu": torch.cuda.get_device_name(0), "steps": a.steps,
                      "reference_ms_per_step": r_ms, "this_package_ms_per_step": o_ms, "speedup": r_ms / o_ms,
                      "reference_max_tokens_per_expert": tight, "rel_err_this_package_vs_reference": errs,
                      "note": "both launched eagerly from Python, one GPU, no expert parallelism"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 5])
    a = ap.parse_args()
    try:
        import flashfusemoe as ref
    except Exception as exc:
        print(json.dumps({"reference_on_gpu": "unavailable", "why": f"{type(exc).__name__}: {str(exc)[:200]}"}))
        return
    import flashfusedmoe_b200 as ffm
    from flashfusedmoe_b200 import ops
    if a.config != 2:
        functional_case(a, ref, ffm, ops)
        return

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    D, F, E, k = 1024, 4096, 8, 2
    torch.manual_seed(1)
    r_layer = ref.MoELayer(D, F, E, k, num_shared_experts=1)
    with torch.no_grad():
        for p in r_layer.parameters():
            p.normal_(0.0, 0.02)
    r_layer = r_layer.to(dev).bfloat16()
    o_layer = ffm.MoELayer(D, F, E, k, num_shared_experts=1).to(dev).bfloat16()
    o_layer.load_state_dict(r_layer.state_dict(), strict=True)
    x = torch.randn(8, 2048, D).bfloat16().to(dev)
    go = torch.randn(8, 2048, D).bfloat16().to(dev).contiguous()

    # the largest per-expert load of this input, from this package's routing (checked against the reference's below)
    with torch.no_grad():
        _, m = ffm.fused_moe(x.view(-1, D), o_layer.gate.weight, o_layer.w_up, o_layer.w_down, top_k=k,
                             return_metrics=True)
    tight = int(m["max_expert_load"])
    r_layer.max_tokens_per_expert = tight   # (allow_dropped_tokens stays True, the layer's default: no host sync)

    def make_step(layer, xin):
        def step():
            for p in layer.parameters():
                p.grad = None
            xin.grad = None
            out, _ = layer(xin)
            out.backward(go)
            return out
        return step

    xr = x.clone().requires_grad_()
    xo = x.clone().requires_grad_()
    r_step, o_step = make_step(r_layer, xr), make_step(o_layer, xo)
    r_ms = timed(r_step, a.steps, a.warmup)
    o_ms = timed(o_step, a.steps, a.warmup)
    r_ms2 = timed(r_step, a.steps, 2)
    o_ms2 = timed(o_step, a.steps, 2)
    ops.check_status()
    out_r, out_o = r_step(), o_step()
    torch.cuda.synchronize()
    # the reference as a user gets it by default: its own estimate of the per-expert bound (twice the balanced load)
    r_layer.max_tokens_per_expert = None
    r_default_ms = timed(r_step, a.steps, a.warmup)
    r_layer.max_tokens_per_expert = tight
    names = [n for n, _ in r_layer.named_parameters()]
    errs = {"out": rel(out_o, out_r), "dH": rel(xo.grad, xr.grad)}
    rp, op_ = dict(r_layer.named_parameters()), dict(o_layer.named_parameters())
    for n in names:
        errs["d " + n] = rel(op_[n].grad, rp[n].grad)
    tokens = x.shape[0] * x.shape[1]
    print(json.dumps({
        "workload": "BASELINE configs[1]: MoELayer(1024, 4096, 8, top_k=2, swiglu, 1 shared expert), x [8, 2048, 1024] "
                    "bf16, seed 1, weights N(0, 0.02), forward + backward, dense grad_output",
        "gpu": torch.cuda.get_device_name(0), "steps": a.steps,
        "reference_ms_per_step": min(r_ms, r_ms2), "this_package_ms_per_step": min(o_ms, o_ms2),
        "reference_ms_per_step_runs": [r_ms, r_ms2], "this_package_ms_per_step_runs": [o_ms, o_ms2],
        "reference_tokens_per_s": tokens / (min(r_ms, r_ms2) * 1e-3),
        "this_package_tokens_per_s": tokens / (min(o_ms, o_ms2) * 1e-3),
        "speedup": min(r_ms, r_ms2) / min(o_ms, o_ms2),
        "reference_max_tokens_per_expert": tight,
        "reference_ms_per_step_default_bound": r_default_ms,
        "rel_err_this_package_vs_reference": errs,
        "note": "both launched eagerly from Python; the reference through its own Triton kernels and cuBLAS bmm"}))


if __name__ == "__main__":
    main()
