"""Throughput of the two larger BASELINE shapes (forward + backward), one process per GPU.

    python -m flashfusedmoe_b200.bench_configs --config 3 [--steps 20] [--warmup 5]
    python -m torch.distributed.run --nproc-per-node N ... -m flashfusedmoe_b200.bench_configs --config 3|4

config 3  Mixtral-shaped layer: D 4096, 8 experts, top-2, swiglu, ffn_dim 2 x 14336, 8192 tokens per GPU, seed 2,
          weights N(0, 0.02), a gate bias log(p_e) with p ~ Zipf(s = 1.1) over a seeded permutation of the experts
          (fp32 `expert_bias`: selection only), fused_moe() called directly with this rank's expert slice.
config 4  fine-grained layer with latent projection: MoELayer(2048, 2816, 64, 6, latent_dim=512, 2 shared experts
          merged into one GLU FFN of ffn_dim 2 x 2816), 16384 tokens per GPU, seed 3, expert parallel only (N >= 2),
          dense gradients through OverlappedGradSync(num_buckets=4).
Synthetic inputs: tokens N(0, 1) seeded per rank, grad_out N(0, 1). Timed with CUDA events after a group barrier,
maximum over ranks; a second pass with per-kernel events gives the grouped-GEMM rate. Rank 0 prints one JSON line.
"""

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import MoELayer, fused_moe, ops, OverlappedGradSync, get_dense_params


def zipf_bias(E, seed, s=1.1):
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(E, generator=g)
    p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** s
    p = p / p.sum()
    bias = torch.empty(E, dtype=torch.float32)
    bias[perm] = torch.log(p).float()
    return bias - bias.mean()


def run(config, steps, warmup, group, rank, world, dev, per_kernel=True):
    """Time `steps` forward + backward passes of one configuration on an initialised process group (or a single
    GPU, group None). Returns the result dict on rank 0 and None elsewhere."""
    a = argparse.Namespace(config=config, steps=steps, warmup=warmup)
    if a.config == 3:
        D, F, E, k, N = 4096, 28672, 8, 2, 8192
        H = F // 2
        e_local = E // world
        torch.manual_seed(2)
        gate = (torch.randn(E, D) * 0.02).bfloat16().to(dev).requires_grad_()
        # only this rank's expert slice is materialised (same generator order on every rank)
        wu = torch.empty(e_local, F, D, dtype=torch.bfloat16, device=dev)
        wd = torch.empty(e_local, D, H, dtype=torch.bfloat16, device=dev)
        for e in range(E):
            u = (torch.randn(F, D) * 0.02).bfloat16()
            d = (torch.randn(D, H) * 0.02).bfloat16()
            if e // e_local == rank:
                wu[e % e_local].copy_(u)
                wd[e % e_local].copy_(d)
        wu.requires_grad_()
        wd.requires_grad_()
        bias = zipf_bias(E, 2).to(dev)
        params = [gate, wu, wd]
        torch.manual_seed(2000 + rank)
        x = torch.randn(N, D).bfloat16().to(dev).requires_grad_()
        go = torch.randn(N, D).bfloat16().to(dev)
        counts_seen = {}

        def step():
            for p in params + [x]:
                p.grad = None
            out, losses = fused_moe(x, gate, wu, wd, top_k=k, expert_bias=bias, ep_group=group, return_metrics=True)
            counts_seen["tpe"] = losses["tokens_per_expert"]
            (out * go).sum(dtype=torch.float32).backward()

        flops = (18.0 if world == 1 else 14.0) * N * k * D * H
        name = "BASELINE configs[2]: D=4096 E=8 top_k=2 swiglu ffn_dim=2x14336, 8192 tokens/GPU, Zipf(1.1) gate bias"
    else:
        if world < 2:
            raise ValueError("config 4 is an expert-parallel configuration: run it under torchrun with N >= 2")
        D, F, E, k, N, L = 2048, 2816, 64, 6, 16384, 512
        H = F // 2
        torch.manual_seed(3)
        layer = MoELayer(D, F, E, k, latent_dim=L, num_shared_experts=2, shared_ffn_dim=2 * F)
        with torch.no_grad():
            for p in layer.parameters():
                p.normal_(0.0, 0.02)
        layer = layer.to(dev).bfloat16()
        layer.shard_experts(group)
        sync = OverlappedGradSync(get_dense_params(layer), group, num_buckets=4)
        torch.manual_seed(3000 + rank)
        x = torch.randn(N, D).bfloat16().to(dev).requires_grad_()
        go = torch.randn(N, D).bfloat16().to(dev)
        counts_seen = {}

        def step():
            for p in layer.parameters():
                p.grad = None
            x.grad = None
            out, _ = layer(x)
            (out * go).sum(dtype=torch.float32).backward()
            sync.finish()

        Hs = F  # merged shared FFN: half width = 2 x 1408 = 2816
        flops = 14.0 * N * k * D * H + 18.0 * N * D * Hs + 2.0 * N * D * L * 3 + 3 * 2.0 * N * k * L * D * 3
        name = ("BASELINE configs[3]: D=2048 latent 512 E=64 top_k=6 swiglu ffn_dim=2x1408, shared FFN 2x2816 merged, "
                "16384 tokens/GPU, OverlappedGradSync(4)")

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(a.warmup, 3)):
        step()
    ops.check_status()
    fence()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(a.steps):
        step()
    t1.record()
    fence()
    ms = t0.elapsed_time(t1)
    timer = ops.KernelTimer()
    if per_kernel:
        ops.set_timer(timer)
        for _ in range(a.steps):
            step()
        fence()
        ops.set_timer(None)
    ops.check_status()
    # config 4: how much of the dense-gradient all-reduce the backward pass hides. The same steps (a) without any
    # gradient synchronisation and (c) with one flat AVG all-reduce of all dense gradients after backward has finished;
    # the overlapped schedule timed above is (b). hidden = 1 - (b - a) / (c - a).
    sync_ms = None
    if a.config == 4:
        sync.remove_hooks()
        dense = get_dense_params(layer)

        def step_plain():
            for p in layer.parameters():
                p.grad = None
            x.grad = None
            out, _ = layer(x)
            (out * go).sum(dtype=torch.float32).backward()

        def step_serial():
            step_plain()
            flat = torch.cat([p.grad.reshape(-1) for p in dense])
            dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=group)
            off = 0
            for p in dense:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                off += p.numel()

        def timed(fn):
            for _ in range(2):
                fn()
            fence()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.steps):
                fn()
            e1.record()
            fence()
            return e0.elapsed_time(e1)

        sync_ms = (timed(step_plain), timed(step_serial))
    t = torch.tensor([ms] + list(sync_ms or (0.0, 0.0)), device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    line = None
    if rank == 0:
        kt = timer.totals_ms()
        gemm_ms = sum(kt[n][1] for n in ("gemm_up_glu", "gemm", "gemm_wgrad") if n in kt)
        line = {"metric": "moe_layer_tokens_per_s_fwd_bwd", "config": name, "n_gpus": world, "steps": a.steps,
                "value": N * world * a.steps / (float(t[0]) * 1e-3), "unit": "tokens/s",
                "ms_per_step": float(t[0]) / a.steps, "dtype": "bf16", "data": "synthetic",
                "algorithmic_gemm_tflop_per_step_per_gpu": flops / 1e12,
                "gemm_tflops_per_gpu_whole_step": flops * a.steps / (float(t[0]) * 1e-3) / 1e12}
        if per_kernel:
            line.update({"gemm_ms_per_step": gemm_ms / a.steps,
                         "gemm_tflops_per_gpu_nominal_flops": (flops * a.steps / (gemm_ms * 1e-3) / 1e12
                                                               if gemm_ms > 0 else None),
                         "kernel_ms_per_step": {n: v[1] / a.steps for n, v in kt.items()}})
        if "tpe" in counts_seen:
            line["tokens_per_expert_rank0"] = counts_seen["tpe"].tolist()
        if sync_ms is not None:
            none_ms, serial_ms = float(t[1]) / a.steps, float(t[2]) / a.steps
            over_ms = float(t[0]) / a.steps
            cost = serial_ms - none_ms
            line["grad_sync"] = {"dense_gradient_bytes": sum(p.numel() for p in dense) * 2,
                                 "ms_per_step_without_sync": none_ms, "ms_per_step_overlapped": over_ms,
                                 "ms_per_step_sync_after_backward": serial_ms,
                                 "hidden_frac": (min(1.0, max(0.0, 1.0 - (over_ms - none_ms) / cost))
                                                 if cost > 0 else None)}
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=[3, 4])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    if a.config == 4 and world < 2:
        raise SystemExit("config 4 is an expert-parallel configuration: run it under torchrun with N >= 2")
    line = run(a.config, a.steps, a.warmup, group, rank, world, dev)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
