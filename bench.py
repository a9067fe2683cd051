"""Benchmark of the fused MoE layer: tokens/s of forward + backward on synthetic data.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched with torch.distributed.run)
    python bench.py --impl reference ...                      the reference algorithm on the host CPU cores

Workload at N = 1: BASELINE configs[1] — MoELayer(d_model 1024, ffn_dim 4096, 8 experts, top-2, swiglu, one shared
expert), x [8, 2048, 1024] bf16, seed 1, all weights N(0, 0.02). At N > 1 the same layer with its experts sharded
over the N ranks (expert parallelism) and 16,384 tokens per rank (weak scaling).

One step = forward, loss = <out, grad_out>, backward to every parameter and to the input.
Prints ONE JSON line on rank 0 (see the keys below).
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "moe_layer_tokens_per_s_fwd_bwd"
UNIT = "tokens/s"
CFG = dict(d_model=1024, ffn_dim=4096, num_experts=8, top_k=2, shared_ffn_dim=4096, batch=8, seq=2048, seed=1)
SMI_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def algorithmic_flops(tokens, ep):
    """FLOPs of one step per GPU, unpadded (T = tokens * k routed rows)."""
    D, H, k, E = CFG["d_model"], CFG["ffn_dim"] // 2, CFG["top_k"], CFG["num_experts"]
    Hs = CFG["shared_ffn_dim"] // 2
    T = tokens * k
    routed_fwd = 6.0 * T * D * H
    routed_bwd = 12.0 * T * D * H if ep == 1 else 8.0 * T * D * H  # EP backward has no expert input gradient
    shared = 18.0 * tokens * D * Hs
    return dict(gemm=routed_fwd + routed_bwd + shared, gate=6.0 * tokens * D * E)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(tflops=p["bf16_tflops_sustained"], tflops_burst=p["bf16_tflops"], hbm_gbs=p["hbm_gbs"],
                    source="measured")
    return dict(tflops=1400.0, tflops_burst=1590.0, hbm_gbs=6650.0, source="fallback")


_SAMPLER_SCRIPT = r"""
import sys, time
import pynvml as nv
nv.nvmlInit()
h = nv.nvmlDeviceGetHandleByUUID(sys.argv[1])
out = open(sys.argv[2], "w")
out.write("max,%d\n" % nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
out.flush()
while True:
    try:
        out.write("%.4f,%d,%.1f,%d\n" % (time.time(), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                                          nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                                          nv.nvmlDeviceGetCurrentClocksEventReasons(h)))
        out.flush()
    except nv.NVMLError:
        pass
    time.sleep(float(sys.argv[3]))
"""


# NVML polling period. Measured on this pool: a poll every 10 ms stalled a step of the timed region by 2-24 ms in
# one run out of three (steps are 1.8 ms), every 100 ms still in two of three, once a second never; 200 ms is the
# period of the `nvidia-smi -lms 200` line it replaces.
SAMPLE_S = float(os.environ.get("FFM_BENCH_SAMPLE_MS", "200")) / 1e3


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU while the timed regions run. Read-only.

    A child process polls NVML every 200 ms from before the warm-up (the device is looked up by the UUID torch
    reports, so CUDA_VISIBLE_DEVICES does not matter) and stamps every sample with the wall clock; begin() and
    stop() bracket the timed regions and only samples between them are used. A child process rather than a thread:
    the step loop is close to CPU-bound at N > 1 and must not share the interpreter lock with the sampler.
    `nvidia-smi -lms 200` is the fallback where the NVML binding is missing."""

    REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
                   ("sw_power_cap", 0x4))

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.mode = None
        self.t_begin = None
        self.path = f"/tmp/ffm_bench_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            import pynvml  # noqa: F401  (only to know whether the child can import it)
            uuid = "GPU-" + str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_SCRIPT, uuid, self.path, str(SAMPLE_S)],
                                         stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
            self.mode = "nvml"
            # wait until the child has initialised NVML and written its first sample: the first NVML initialisation on
            # a box takes a while and stalls kernel launches of other processes while it runs
            deadline = time.time() + 15.0
            while time.time() < deadline and self.proc.poll() is None:
                try:
                    if sum(1 for _ in open(self.path)) >= 2:
                        break
                except OSError:
                    pass
                time.sleep(0.05)
            return
        except Exception:
            self.proc = None
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={SMI_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
            self.mode = "smi"
        except OSError:
            self.proc = None

    def begin(self):
        self.t_begin = time.time()

    def _end_child(self):
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()

    def stop(self):
        t_end = time.time()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        if self.mode == "nvml":
            self._end_child()
            sm_max, samples = None, []
            try:
                for line in open(self.path):
                    f = line.strip().split(",")
                    if f[0] == "max":
                        sm_max = float(f[1])
                    elif len(f) == 4 and (self.t_begin or 0.0) <= float(f[0]) <= t_end:
                        samples.append((int(f[1]), float(f[2]), int(f[3])))
                os.remove(self.path)
            except (OSError, ValueError):
                pass
            if sm_max is not None and samples:
                sm = [s[0] for s in samples]
                busy = [s[0] for s in samples if s[1] >= 300.0] or sm   # samples taken while the GPU drew real power
                mask = 0
                for s in samples:
                    mask |= s[2]
                return {"sm_mhz": statistics.median(busy), "sm_max_mhz": sm_max, "sm_mhz_min": min(sm),
                        "power_w_max": max(s[1] for s in samples), "samples": len(sm), "samples_under_load": len(busy),
                        "source": f"nvml, child process, {SAMPLE_S * 1e3:.0f} ms",
                        "reasons": sorted(n for n, bit in self.REASON_BITS if mask & bit)}
            return {"sm_mhz": None, "sm_max_mhz": sm_max, "samples": 0, "reasons": ["no NVML samples in the timed window"]}
        time.sleep(0.25)
        self._end_child()
        self.out.close()
        sm, smax, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "source": "nvidia-smi 200 ms", "reasons": sorted(reasons)}


def build_layer(device, ep_group):
    import flashfusedmoe_b200 as ffm
    torch.manual_seed(CFG["seed"])
    layer = ffm.MoELayer(CFG["d_model"], CFG["ffn_dim"], CFG["num_experts"], CFG["top_k"], num_shared_experts=1,
                         shared_ffn_dim=CFG["shared_ffn_dim"])
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0.0, 0.02)   # same generator order on every rank: weights are replicated before sharding
    layer = layer.to(device).bfloat16()
    if ep_group is not None:
        layer.shard_experts(ep_group)
    return layer


def layer_counts(layer, x):
    """Rows this rank routes to every expert (int64 [E], host) for input x."""
    from flashfusedmoe_b200 import ops
    xf = x.detach().reshape(-1, x.shape[-1])
    r = ops.route_forward(xf, layer.gate.weight.detach(), layer.top_k, layer.gating)
    return r.counts.to(torch.int64).cpu()


def make_step(layer, x, go):
    def step():
        for p in layer.parameters():
            p.grad = None
        x.grad = None
        out, _ = layer(x)
        out.backward(go)
    return step


def capture_step(fn, warm=2):
    """fn() captured into a CUDA graph after `warm` eager runs on a side stream. Every stream the step forks to is
    joined again before it returns, so the whole forward + backward becomes one graph. Returns (graph, kernels of
    this library per replay)."""
    from flashfusedmoe_b200 import ops
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    n0 = ops.launch_count
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    torch.cuda.synchronize()
    return graph, ops.launch_count - n0


def oracle_sample_tokens_per_s(sample_tokens, threads, repeats=1):
    """The oracle's forward + backward (the reference algorithm restated on CPU, fp32 accumulation, bf16 rounding
    points) on a token sub-sample of the same workload; returns (tokens/s, seconds per pass)."""
    from oracle import moe_oracle as orc
    torch.set_num_threads(threads)
    torch.manual_seed(CFG["seed"])
    D, F, E, k = CFG["d_model"], CFG["ffn_dim"], CFG["num_experts"], CFG["top_k"]
    Hs = CFG["shared_ffn_dim"] // 2
    g = (torch.randn(E, D) * 0.02).bfloat16()
    wu = (torch.randn(E, F, D) * 0.02).bfloat16()
    wd = (torch.randn(E, D, F // 2) * 0.02).bfloat16()
    sg, su = (torch.randn(Hs, D) * 0.02).bfloat16(), (torch.randn(Hs, D) * 0.02).bfloat16()
    sd = (torch.randn(D, Hs) * 0.02).bfloat16()
    h = torch.randn(sample_tokens, D).bfloat16()
    go = torch.randn(sample_tokens, D).bfloat16()
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        fw = orc.fused_moe_forward(h, g, wu, wd, k, "swiglu", "softmax", dtype=torch.bfloat16)
        orc.fused_moe_backward(fw, go)
        # shared expert forward + backward (same GLU FFN arithmetic, one group)
        pre = torch.cat([orc.mm(h, sg.T, torch.bfloat16), orc.mm(h, su.T, torch.bfloat16)], -1)
        act = orc.glu_forward(pre, "swiglu", torch.bfloat16)
        orc.mm(act, sd.T, torch.bfloat16)
        d_act = orc.mm(go, sd, torch.bfloat16)
        gU = orc.glu_backward(d_act, pre, "swiglu", torch.bfloat16)
        orc.mm(gU, torch.cat([sg, su], 0), torch.bfloat16)
        orc.mm(gU.T, h, torch.bfloat16)
        orc.mm(go.T, act, torch.bfloat16)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return sample_tokens / best, best



def _rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def routing_only_input_grad(x, go, gate, w_up, w_down, shared, idx):
    """fp32 autograd restatement (on the GPU) of the input gradient the expert-parallel backward returns: the
    routing-weight path and the shared expert, with the experts' own input treated as a constant (the reference's
    contract, src/flashfusemoe/fused_moe.py:1001-1005). `idx` [n, k] are the kernel's expert assignments."""
    F = torch.nn.functional
    n, D = x.shape
    E = gate.shape[0]
    H = w_up.shape[1] // 2
    xf = x.float().requires_grad_()
    w = torch.softmax((xf @ gate.float().T).gather(1, idx.long()), dim=-1)
    xd = x.float()
    routed = torch.zeros(n, D, device=x.device)
    for e in range(E):
        rows, slot = (idx == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        pre = xd[rows] @ w_up[e].float().T
        y = (F.silu(pre[:, :H]) * pre[:, H:]) @ w_down[e].float().T
        routed = routed.index_add(0, rows, w[rows, slot].unsqueeze(1) * y)
    sg, su, sd = (t.float() for t in shared)
    dense = (F.silu(xf @ sg.T) * (xf @ su.T)) @ sd.T
    ((routed + dense) * go.float()).sum().backward()
    return xf.grad


def ep_parity_check(device, group, rank, world, tokens=2048):
    """Expert-parallel layer against this package's single-GPU layer on the same tokens and the same (unsharded)
    weights, outside every timed region; mirrors the reference's tests/test_multigpu.py:96-212. Every rank draws
    its own tokens. Returns a dict of the worst figures over all ranks with "ok"."""
    import torch.distributed as dist
    import flashfusedmoe_b200 as ffm
    from flashfusedmoe_b200 import ops
    fm = sys.modules["flashfusedmoe_b200.fused_moe"]
    k, E, D = CFG["top_k"], CFG["num_experts"], CFG["d_model"]
    full = build_layer(device, None)
    sharded = build_layer(device, group)          # same seed, same weights; keeps this rank's experts
    el = E // world
    torch.manual_seed(CFG["seed"] + 5000 + rank)
    x = torch.randn(tokens, D, device=device).bfloat16()
    go = torch.randn(tokens, D, device=device).bfloat16()

    def shared_of(layer):
        se = layer.shared_expert
        return (se.w_gate.weight, se.w_up.weight, se.w_down.weight)

    xe = x.clone().requires_grad_()
    out_e, m_e = ffm.fused_moe(xe, sharded.gate.weight, sharded.w_up, sharded.w_down, top_k=k, ep_group=group,
                               shared_expert_weights=shared_of(sharded), return_metrics=True)
    out_e.backward(go)
    ops.check_status()
    # the same tokens through the single-GPU path with the full weights
    ffm.set_ep_group(None)
    xs = x.clone().requires_grad_()
    addend = fm.glu_ffn(xs, *shared_of(full))
    out_1, m_1 = ffm.fused_moe(xs, full.gate.weight, full.w_up, full.w_down, top_k=k, return_metrics=True,
                               _addend=addend)
    out_1.backward(go)
    idx = ops.route_forward(x, full.gate.weight.detach(), k).topk_idx
    ops.check_status()
    ffm.set_ep_group(group)
    # expert weight gradients: summed over every rank's tokens and scaled by 1 / ep (fused_moe.py:961-966)
    g_up, g_down = full.w_up.grad.float().clone(), full.w_down.grad.float().clone()
    dist.all_reduce(g_up, group=group)
    dist.all_reduce(g_down, group=group)
    dh_ref = routing_only_input_grad(x, go, full.gate.weight.detach(), full.w_up.detach(), full.w_down.detach(),
                                     [t.detach() for t in shared_of(full)], idx)
    res = {
        "counts_equal": float(torch.equal(m_e["tokens_per_expert"], m_1["tokens_per_expert"])),
        "out": _rel(out_e, out_1),
        "dW_up": _rel(sharded.w_up.grad, g_up[rank * el:(rank + 1) * el] / world),
        "dW_down": _rel(sharded.w_down.grad, g_down[rank * el:(rank + 1) * el] / world),
        "dGate": _rel(sharded.gate.weight.grad, full.gate.weight.grad),
        "dW_shared": max(_rel(a.grad, b.grad) for a, b in zip(shared_of(sharded), shared_of(full))),
        "dH": _rel(xe.grad, dh_ref),
    }
    t = torch.tensor([res["out"], res["dW_up"], res["dW_down"], res["dGate"], res["dW_shared"], res["dH"],
                      1.0 - res["counts_equal"]], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    out, dwu, dwd, dg, dws, dh, cnt_bad = (float(v) for v in t)
    tol = {"out": 1e-6, "dW_up": 2e-2, "dW_down": 2e-2, "dGate": 1e-3, "dW_shared": 1e-6, "dH": 2e-2}
    worst = {"out": out, "dW_up": dwu, "dW_down": dwd, "dGate": dg, "dW_shared": dws, "dH": dh}
    ok = cnt_bad == 0.0 and all(worst[n] <= tol[n] for n in tol)
    del full, sharded
    torch.cuda.empty_cache()
    return {"ok": bool(ok), "counts_equal": cnt_bad == 0.0, **worst, "tolerance": tol, "tokens_per_rank": tokens,
            "against": "single-GPU path of this package on the same tokens and unsharded weights (out, dW, dGate, "
                       "counts); fp32 autograd restatement on the GPU for the routing-only + shared-expert dH; "
                       "maximum over ranks of max|a-b| / max|b|"}


def measure_peer_copy(group, device, rank, world, nbytes=256 << 20, repeats=5):
    """NVLink bandwidth per direction while every rank copies `nbytes` to its right-hand neighbour at once: with the
    copy engine (torch copy_ into the neighbour's symmetric buffer) and with this library's plain-store push kernel.
    Returns GB/s (best of `repeats`, maximum time over ranks), or None when symmetric memory is unavailable."""
    import ctypes
    import torch.distributed as dist
    from flashfusedmoe_b200 import _lib, ops
    try:
        import torch.distributed._symmetric_memory as symm_mem
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        hdl = symm_mem.rendezvous(buf, group)
        nxt = (rank + 1) % world
        peer = hdl.get_buffer(nxt, (nbytes,), torch.uint8)
        peer_ptr = int(hdl.buffer_ptrs[nxt])
    except Exception as exc:  # no symmetric memory on this build
        return {"unavailable": str(exc)[:200]}
    src = torch.empty(nbytes, dtype=torch.uint8, device=device).random_(0, 255)
    lib = _lib.load()

    def best_ms(fn):
        best = None
        for _ in range(repeats + 1):
            torch.cuda.synchronize()
            dist.barrier(group)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b)
            best = ms if best is None else min(best, ms)
        t = torch.tensor([best], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t[0])

    def push():
        srcs = (ctypes.c_void_p * 1)(src.data_ptr())
        dsts = (ctypes.c_void_p * 1)(peer_ptr)
        sizes = (ctypes.c_int64 * 1)(nbytes)
        _lib.check(lib.ffm_p2p_push(1, srcs, dsts, sizes, ops._stream()), "ffm_p2p_push")

    copy_ms = best_ms(lambda: peer.copy_(src, non_blocking=True))
    push_ms = best_ms(push)
    torch.cuda.synchronize()
    dist.barrier(group)
    del peer, hdl, buf
    return {"bytes": nbytes, "copy_engine_gbs": nbytes / (copy_ms * 1e-3) / 1e9,
            "push_kernel_gbs": nbytes / (push_ms * 1e-3) / 1e9,
            "pattern": "every rank to its right-hand neighbour at the same time, per direction"}


def other_configs(group, rank, world, device):
    """The other BASELINE shapes, a few steps each: configs[2] (Mixtral-shaped, Zipf gate bias) and, expert parallel
    only, configs[3] (fine-grained with latent projection) as tokens/s forward + backward; configs[4] (decode shape,
    forward only) as p50 / p99 latency, eager and replayed from a CUDA graph. Rank 0 gets the dict."""
    from flashfusedmoe_b200 import bench_configs, bench_decode
    out = {}
    try:
        out["configs[2]"] = bench_configs.run(3, 6, 3, group, rank, world, device, per_kernel=False)
        torch.cuda.empty_cache()
        if world > 1:
            out["configs[3]"] = bench_configs.run(4, 8, 3, group, rank, world, device, per_kernel=False)
            torch.cuda.empty_cache()
        else:
            out["configs[3]"] = {"skipped": "expert-parallel configuration (latent projection around the exchange): N >= 2"}
        out["configs[4]_eager"] = bench_decode.run(60, 10, 128, False, group, rank, world, device)
        torch.cuda.empty_cache()
        out["configs[4]_graph"] = bench_decode.run(60, 10, 128, True, group, rank, world, device)
        torch.cuda.empty_cache()
        if world == 1:
            out["configs[1]_fp8_forward"] = fp8_forward_steps(device)
            torch.cuda.empty_cache()
    except Exception as exc:   # the headline line must still be printed
        out["error"] = f"{type(exc).__name__}: {str(exc)[:300]}"
    if rank != 0:
        return None
    keep = ("value", "unit", "ms_per_step", "gemm_tflops_per_gpu_whole_step", "p50", "p99", "min", "mode",
            "weight_stream_bound_ms", "tokens_per_gpu", "iters", "steps", "config", "skipped", "grad_sync", "all_to_all_ms_per_iter")
    return {n: ({k: v for k, v in d.items() if k in keep} if isinstance(d, dict) else d) for n, d in out.items()}


def fp8_forward_steps(device, steps=12, warmup=4):
    """configs[1] on one GPU with the opt-in e4m3 forward projections of the routed experts (backward stays bf16):
    the same step as the headline, captured and replayed, a few steps."""
    import flashfusedmoe_b200 as ffm
    layer = build_layer(device, None)
    torch.manual_seed(1000)
    x = torch.randn(CFG["batch"], CFG["seq"], CFG["d_model"], device=device).bfloat16().requires_grad_()
    go = torch.randn_like(x)
    step = make_step(layer, x, go)
    ffm.set_expert_gemm_precision("fp8")
    try:
        graph, _ = capture_step(step)
        for _ in range(warmup):
            graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
    finally:
        ffm.set_expert_gemm_precision("bf16")
    tokens = CFG["batch"] * CFG["seq"]
    return {"config": "BASELINE configs[1] with e4m3 operands in the routed experts' forward GEMMs (activations scaled "
                      "per row, weights per expert; opt-in, not the headline precision), replayed graph",
            "steps": steps, "value": tokens / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = 2048
    # warm-up passes and timed steps, each step one bounded sample of the workload
    for _ in range(max(args.warmup, 1)):
        oracle_sample_tokens_per_s(256, threads)
    vals = [oracle_sample_tokens_per_s(sample, threads)[0] for _ in range(args.steps)]
    v = statistics.median(vals)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * sample / v, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "BASELINE configs[1]: MoELayer d_model=1024 ffn_dim=4096 E=8 top_k=2 swiglu + 1 shared expert, "
                                   "fwd+bwd; reference algorithm on host CPU cores"},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"{sample} of 16384 tokens per step, same layer shape; the Python/Triton reference "
                                       "cannot travel to the GPU box, its CPU restatement (oracle/) is timed"},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--launch", default="graph", choices=["graph", "eager"],
                    help="graph: the step is captured once into a CUDA graph and the timed regions replay it (the "
                         "launch thread then cannot starve the GPU); eager: every kernel launched from Python. "
                         "Falls back to eager where the step cannot be captured (it reads counts on the host).")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the seconds-long sustained region and the other BASELINE configurations")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch.distributed as dist
    from flashfusedmoe_b200 import ops

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    W = max(args.warmup, 3)
    K = args.steps

    # ---- expert parallel only: numerics of the sharded layer against the single-GPU path, before anything is timed
    ep_parity = nvlink = None
    tokens = CFG["batch"] * CFG["seq"]
    # Host-sync-free expert parallelism (set_ep_static_forward): buffers sized for the worst case, exchange tables built
    # on the device, no host read of the routing counts, so the training step can be captured into a CUDA graph like
    # the single-GPU one. FFM_BENCH_EP_STATIC=0 measures the host-planned path (one host sync per call, eager only).
    ep_static = world > 1 and os.environ.get("FFM_BENCH_EP_STATIC", "1") != "0"
    if ep_static:
        import flashfusedmoe_b200 as _ffm
        _ffm.set_ep_static_forward(tokens)
    if world > 1:
        ep_parity = ep_parity_check(device, group, rank, world)
        nvlink = measure_peer_copy(group, device, rank, world)

    layer = build_layer(device, group)
    torch.manual_seed(CFG["seed"] + 1000 + rank)  # different tokens on every rank
    x_host = torch.randn(CFG["batch"], CFG["seq"], CFG["d_model"]).bfloat16().pin_memory()
    go = torch.randn(CFG["batch"], CFG["seq"], CFG["d_model"], device=device).bfloat16()
    x = x_host.to(device).requires_grad_()
    step = make_step(layer, x, go)

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident timing --------------------------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()   # the child starts polling during the warm-up; only samples after begin() count
    for _ in range(W):
        step()
    ops.check_status()
    timer = ops.KernelTimer()
    # The eager launch loop runs only a step or so ahead of the GPU right after the fence, so a pause of the launching
    # thread (a descheduled process on a shared host, the garbage collector, a driver lock taken by a monitoring
    # call) shows up as a stalled step. A captured step has no such dependence: K replays are queued at once.
    import gc
    gc.collect()
    gc.disable()
    graph = None
    graph_note = None
    launches_per_replay = 0
    can_capture = world == 1 or ep_static   # the host-planned expert-parallel step reads the row counts on the host
    if args.launch == "graph" and can_capture:
        try:
            graph, launches_per_replay = capture_step(step)
        except Exception as exc:   # keep measuring, eagerly
            graph, graph_note = None, f"capture failed: {type(exc).__name__}: {str(exc)[:200]}"
            torch.cuda.synchronize()
    elif args.launch == "graph":
        graph_note = "not capturable: the host-planned expert-parallel step reads the row counts on the host"
    run_step = graph.replay if graph is not None else step
    graph_used = graph is not None
    # Capturing executes nothing, so ranks leave it at different times; a rank that replayed at once would sit in the
    # exchange's bounded flag wait while its peer is still capturing. Nobody replays before everybody has captured.
    fence()

    def timed_region(fn):
        fence()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(K - 1)]  # per-step marks: a view into the region
        a.record()
        for i in range(K):
            fn()
            if i < K - 1:
                marks[i].record()
        b.record()
        fence()
        edges = [a] + marks + [b]
        return a.elapsed_time(b), [edges[i].elapsed_time(edges[i + 1]) for i in range(K)]

    for _ in range(2):
        run_step()
    fence()   # (every rank: the fence holds a collective)
    if sampler:
        sampler.begin()
    launches0 = ops.launch_count
    ms, step_series = timed_region(run_step)
    launches = (ops.launch_count - launches0) if graph is None else launches_per_replay * K
    step_ms = sorted(step_series)
    ops.check_status()
    eager = None
    eager_ms = 0.0
    if graph is not None:
        # the same K steps launched kernel by kernel from Python, for comparison (not the reported value)
        time.sleep(0.3)
        for _ in range(2):
            step()
        eager_ms, eager_series = timed_region(step)
        eager = {"value": tokens * world * K / (eager_ms * 1e-3), "unit": UNIT, "ms_per_step": eager_ms / K,
                 "step_ms_median": sorted(eager_series)[K // 2], "step_ms_max": max(eager_series)}

    # ---- per-kernel pass: the same K steps again with a CUDA-event pair around every launch of this library ----
    # (kept out of the timed region above: the ~60 extra event records per step cost about 5 % of a 2 ms step)
    # Same schedule as the timed region: same streams, and the GLU backward riding inside the dW_down GEMM launch,
    # whose event pair therefore times that whole launch against dW_down's FLOPs alone. An event pair around an
    # HBM-bound kernel that shares the GPU with a GEMM of another stream times the sharing, so the figures of the
    # non-GEMM kernels are upper bounds.
    time.sleep(0.5)   # let the board recover the power headroom the timed region started with
    for _ in range(2):
        step()
    a2a_bytes0 = ops.a2a_bytes_sent
    ops.set_timer(timer)
    for _ in range(K):
        step()
    fence()
    ops.set_timer(None)
    a2a_bytes = ops.a2a_bytes_sent - a2a_bytes0
    if ep_static:
        # the host never sees the counts in this mode: one extra call tells how many of this rank's routed rows leave
        # it; a step moves them three times (dispatch, combine, backward)
        el = CFG["num_experts"] // world
        tpe = layer_counts(layer, x)
        remote_rows = int(tpe.sum() - tpe[rank * el:(rank + 1) * el].sum())
        a2a_bytes = 3 * K * remote_rows * CFG["d_model"] * 2

    # ---- expert parallel only: K steps whose row exchanges move nothing (everything else runs) -----------------
    # step time minus this = the exchange time that compute did not hide
    dry_ms = None
    dry_mode = None
    if world > 1:
        fm = sys.modules["flashfusedmoe_b200.fused_moe"]
        fm.set_ep_dry_exchange(True)
        dry_fn = step
        if graph is not None:
            # compared like with like: the dry step is captured and replayed as the measured one is
            try:
                dry_graph, _ = capture_step(step)
                dry_fn, dry_mode = dry_graph.replay, "replayed"
            except Exception:
                torch.cuda.synchronize()
        fence()
        for _ in range(2):
            dry_fn()
        dry_ms, _ = timed_region(dry_fn)
        fm.set_ep_dry_exchange(False)
        if dry_mode is None:
            dry_mode = "eager"
        else:
            del dry_graph
        dry_fn = None
        step()   # one real step: the receive buffers hold real rows again
        fence()

    # ---- end to end: pinned host input in, loss scalar out, every step ------------------------
    # The loop a training script would run around the public API: the next step's input is uploaded on a copy
    # stream while the current step computes (two device buffers), and each step's loss is copied to pinned
    # host memory and read two steps later, so neither transfer stalls the compute stream. Every step still
    # moves its own input host -> device and its own loss device -> host inside the timed region.
    copy_stream = torch.cuda.Stream(device=device)
    x_bufs = [torch.empty_like(x_host, device=device) for _ in range(2)]
    LAG = 2   # a step's loss is read two steps later: the host stays two replays ahead of the GPU
    loss_host = torch.zeros(LAG + 1, dtype=torch.float32).pin_memory()
    uploaded = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    loss_ready = [torch.cuda.Event() for _ in range(LAG + 1)]

    def upload(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])
            x_bufs[i % 2].copy_(x_host, non_blocking=True)
            uploaded[i % 2].record(copy_stream)

    e2e_graph = None
    x_in = torch.empty_like(x).requires_grad_()
    loss_cell = [None]

    def e2e_body():
        for p in layer.parameters():
            p.grad = None
        x_in.grad = None
        out, _ = layer(x_in)
        loss = (out * go).sum(dtype=torch.float32)
        loss.backward()
        loss_cell[0] = loss.detach().reshape(1)

    if graph is not None:
        try:
            with torch.no_grad():
                x_in.copy_(x)
            e2e_graph, _ = capture_step(e2e_body)
        except Exception as exc:
            e2e_graph = None
            graph_note = f"end-to-end capture failed: {type(exc).__name__}: {str(exc)[:200]}"
            torch.cuda.synchronize()
    fence()

    def e2e_run(steps):
        losses_read = []
        main = torch.cuda.current_stream()
        for ev in consumed:
            ev.record(main)
        upload(0)
        for i in range(steps):
            if i + 1 < steps:
                upload(i + 1)
            main.wait_event(uploaded[i % 2])
            if e2e_graph is not None:
                # the graph reads a fixed input buffer: this step's upload is moved into it on the device
                with torch.no_grad():
                    x_in.copy_(x_bufs[i % 2])
                consumed[i % 2].record(main)
                e2e_graph.replay()
                loss = loss_cell[0]
            else:
                for p in layer.parameters():
                    p.grad = None
                xd = x_bufs[i % 2].detach().requires_grad_()
                out, _ = layer(xd)
                loss = (out * go).sum(dtype=torch.float32)
                loss.backward()
                consumed[i % 2].record(main)
                loss = loss.detach().reshape(1)
            slot = i % (LAG + 1)
            loss_host[slot:slot + 1].copy_(loss, non_blocking=True)
            loss_ready[slot].record(main)
            if i >= LAG:
                back = (i - LAG) % (LAG + 1)
                loss_ready[back].synchronize()
                losses_read.append(float(loss_host[back]))
        for i in range(max(steps - LAG, 0), steps):
            back = i % (LAG + 1)
            loss_ready[back].synchronize()
            losses_read.append(float(loss_host[back]))
        return losses_read

    time.sleep(0.5)   # the same power headroom as the device-resident region started with
    e2e_run(3)
    fence()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    read = e2e_run(K)
    e1.record()
    fence()
    assert len(read) == K and all(v == v for v in read)
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None  # sampled from the start of the timed region to here

    # ---- sustained: the same step for at least two seconds (the board settles at its power cap) -------------------
    sus_ms, sus_steps, sus_clocks = 0.0, 0, None
    if not args.no_extras:
        med = torch.tensor([step_ms[K // 2]], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(med, op=dist.ReduceOp.MAX)   # every rank must run the same number of steps
        sus_steps = max(K, int(2600.0 / max(float(med[0]), 1e-3)) + 1)
        sampler2 = ClockSampler(local_rank) if rank == 0 else None
        if sampler2:
            sampler2.start()
        fence()
        if sampler2:
            sampler2.begin()
        s0 = torch.cuda.Event(enable_timing=True)
        s1 = torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(sus_steps):
            run_step()
        s1.record()
        fence()
        sus_ms = s0.elapsed_time(s1)
        sus_clocks = sampler2.stop() if sampler2 else None
        ops.check_status()
    gc.enable()

    t = torch.tensor([ms, e2e_ms, dry_ms if dry_ms is not None else 0.0, sus_ms, eager_ms], device=device,
                     dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, dry_ms, sus_ms, eager_ms = (float(v) for v in t)
    if eager is not None:
        eager.update(value=tokens * world * K / (eager_ms * 1e-3), ms_per_step=eager_ms / K)

    # ---- the other BASELINE configurations, a few steps each, after every timed region of the headline workload ----
    other = None
    if not args.no_extras:
        del layer, step, x, go, x_bufs, x_in, graph, e2e_graph, run_step
        loss_cell[0] = None
        if ep_static:
            _ffm.set_ep_static_forward(None)   # the other configurations choose their own mode (worst-case buffers
                                               # declared for 16,384 tokens would be far too large for them)
        torch.cuda.empty_cache()
        other = other_configs(group, rank, world, device)

    if rank == 0:
        peaks = measured_peaks()
        fl = algorithmic_flops(tokens, world)
        kt = timer.totals_ms()
        gemm_names = ("gemm_up_glu", "gemm", "gemm_wgrad")
        # GEMM launches sit on several streams and two of them never share an SM: the merged intervals of their event
        # pairs are the time the GEMM kernel had the GPU (the plain sum counts a launch queued behind another twice)
        gemm_ms = timer.union_ms(gemm_names)
        gemm_ms_sum = sum(kt[n][1] for n in gemm_names if n in kt)
        gemm_launches = sum(kt[n][0] for n in gemm_names if n in kt)
        achieved = fl["gemm"] * K / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        # the launches that also do the GLU backward (in the dAct GEMM's epilogue, or as a passenger of the dW_down GEMM
        # with FFM_FUSED_GLU_BACKWARD=0): their event time is the whole launch, their FLOPs are the GEMM's alone
        carriers = [n for n in ("gemm_dact_glu_backward", "gemm_wgrad_passenger") if n in kt]
        pass_ms = timer.union_ms(carriers)
        value = tokens * world * K / (ms * 1e-3)
        sm_mhz = (clocks or {}).get("sm_mhz")
        sm_max = (clocks or {}).get("sm_max_mhz")
        # the hardware's dense bf16 rate at the clock sampled during the timed regions (2250 TFLOP/s at the maximum)
        hw_rate = 2250.0 * sm_mhz / sm_max if sm_mhz and sm_max else None
        D_, H_, k_ = CFG["d_model"], CFG["ffn_dim"] // 2, CFG["top_k"]
        rows_ = tokens * k_   # routed rows a GPU's grouped GEMMs see (balanced routing)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "step_ms_median": step_ms[K // 2], "step_ms_max": step_ms[-1],
            "step_ms_first3": step_series[:3], "step_ms_last3": step_series[-3:],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "BASELINE configs[1]: MoELayer d_model=1024 ffn_dim=4096 E=8 top_k=2 swiglu + 1 shared "
                                   "expert (ffn_dim 4096), x [8,2048,1024] bf16 seed 1, weights N(0,0.02), forward+backward",
                       "tokens_per_gpu": tokens, "expert_parallel": world,
                       "launch": ("one forward + backward step captured into a CUDA graph, replayed K times"
                                  if graph_used else "eager: every kernel launched from Python"),
                       "launch_note": graph_note,
                       "expert_parallel_mode": (None if world == 1 else
                                                "host-sync-free (set_ep_static_forward)" if ep_static else
                                                "host-planned (one host read of the routing counts per call)"),
                       "l2": "no explicit flush: one step streams > 1 GB of activations and weights, 8x the 126 MB L2"},
            "e2e": {"value": tokens * world * K / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {
                # the timed regions are sub-second bursts, so the burst cuBLAS figure is the denominator
                "bound": "tensor", "achieved": achieved, "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                "frac": (achieved / peaks["tflops_burst"]) if achieved else None,
                # not captured by this run (ncu is never in a timed run); the ncu figures are in the profile summaries
                "traffic": None,
                # what the largest grouped-GEMM launch of a step (up-projection + GLU of the routed experts) must
                # move: grouped rows x D in, weights in, activations and pre-activations out
                "algorithmic_bytes_largest_launch": 2.0 * (rows_ * D_ + CFG["num_experts"] // world * 2 * H_ * D_
                                                           + rows_ * 3 * H_),
                "kernel": "ffm_gemm_kernel (tcgen05 grouped GEMM, all instantiations)",
                "measured_in": "a second pass of the same K steps after the timed region, same streams and same "
                               "kernels as the timed region, with a CUDA-event pair around every kernel launch of "
                               "the library; GEMM time = merged intervals of the GEMM launches' event pairs (they sit "
                               "on several streams and never share an SM)",
                "peak_source": f"{peaks['source']} cuBLAS bf16 burst (sustained {peaks['tflops']})",
                "frac_of_burst": (achieved / peaks["tflops_burst"]) if achieved else None,
                "frac_of_sustained": (achieved / peaks["tflops"]) if achieved else None,
                "frac_of_nominal_2250": (achieved / 2250.0) if achieved else None,
                "frac_of_hw_rate_at_sampled_clock": (achieved / hw_rate) if achieved and hw_rate else None,
                "whole_step_tflops": fl["gemm"] * K / (ms * 1e-3) / 1e12,
                "glu_backward_schedule": ("epilogue of the dAct GEMM" if "gemm_dact_glu_backward" in carriers else
                                          "passenger warps of the dW_down GEMM" if carriers else None),
                # merged intervals of those launches' event pairs (includes time they wait behind another GEMM)
                "glu_backward_launch_ms_per_step": pass_ms / K,
                "gemm_launches": gemm_launches, "gemm_ms_per_step": gemm_ms / K,
                "gemm_event_pair_sum_ms_per_step": gemm_ms_sum / K,
                "algorithmic_tflop_per_step": fl["gemm"] / 1e12,
                "other_kernels_ms_per_step": {n: v[1] / K for n, v in kt.items()
                                              if n not in gemm_names and n not in ("all_to_all", "exchange_rows", "gemm_wgrad_passenger",
                                                                                  "gemm_dact_glu_backward")},
            },
        }
        if eager is not None:
            line["eager"] = eager
        if sus_steps:
            line["sustained"] = {"value": tokens * world * sus_steps / (sus_ms * 1e-3), "unit": UNIT,
                                 "steps": sus_steps, "seconds": sus_ms * 1e-3, "ms_per_step": sus_ms / sus_steps,
                                 "whole_step_tflops": fl["gemm"] * sus_steps / (sus_ms * 1e-3) / 1e12,
                                 "clocks": sus_clocks}
        if ep_parity is not None:
            line["ep_parity"] = ep_parity
        if other is not None:
            line["other_configs"] = other
        if world > 1 and "all_to_all" in kt:
            # expert-parallel exchange on this rank: three all-to-alls per step (dispatch, combine, backward).
            # Time is from CUDA events around each call on its issuing stream, so it includes waiting for peers;
            # the NVLink fraction is against the per-direction peer copy measured by this run (measure_peer_copy).
            n_a2a, a2a_ms = kt["all_to_all"]
            # the step the dry one is compared with: the replayed one if the dry step was replayed too
            ref_ms = ms if (dry_mode == "replayed" or eager is None) else eager["ms_per_step"] * K
            gbs = a2a_bytes / (a2a_ms * 1e-3) / 1e9 if a2a_ms > 0 else None
            link = (nvlink or {}).get("copy_engine_gbs")
            # the row kernels alone (no barriers, no waiting for peers): what the stores achieve over NVLink; their
            # launches also move this rank's local rows, which the byte count leaves out
            rows_ms = kt["exchange_rows"][1] if "exchange_rows" in kt else None
            rows_gbs = a2a_bytes / (rows_ms * 1e-3) / 1e9 if rows_ms else None
            line["expert_parallel"] = {"all_to_all_calls_per_step": n_a2a / K, "all_to_all_ms_per_step": a2a_ms / K,
                                       "bytes_sent_per_step": a2a_bytes / K, "achieved_gbs_per_direction": gbs,
                                       "row_kernels_ms_per_step": (rows_ms / K) if rows_ms else None,
                                       "row_kernels_gbs_per_direction": rows_gbs,
                                       "row_kernels_frac_of_measured_peer_copy": (rows_gbs / link) if rows_gbs and link else None,
                                       "nvlink_peer_copy": nvlink,
                                       "nvlink_frac_of_measured_peer_copy": (gbs / link) if gbs and link else None,
                                       "nvlink_frac_of_nominal_900": (gbs / 900.0) if gbs else None,
                                       "note": ("E = 8 experts over 8 ranks: one local expert per rank, the "
                                                "degenerate case of this weak-scaling workload" if world == 8 else None),
                                       "share_of_step_in_kernel_pass": (a2a_ms / K) / (ms / K),
                                       # exposed = step time minus the time of the same step with exchanges that move
                                       # nothing; hidden = 1 - exposed / (event time of the exchanges)
                                       "ms_per_step_without_exchange_payload": dry_ms / K,
                                       "dry_step_launch": dry_mode,
                                       "exposed_exchange_ms_per_step": max(0.0, (ref_ms - dry_ms) / K),
                                       "hidden_frac": (min(1.0, max(0.0, 1.0 - (ref_ms - dry_ms) / a2a_ms))
                                                       if a2a_ms > 0 else None),
                                       "transport": os.environ.get("FFM_EP_TRANSPORT", "p2p")}
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, secs = oracle_sample_tokens_per_s(2048, threads, repeats=2)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"2048 of 16384 tokens, same layer shape, oracle fwd+bwd, {secs:.2f} s per pass"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if ep_parity is not None and not ep_parity["ok"]:
        sys.exit(1)   # the throughput of a layer whose numbers are wrong is not a result


if __name__ == "__main__":
    main()
