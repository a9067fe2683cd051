"""Latency of the decode-shaped layer (BASELINE configs[4]): forward only, 128 tokens per GPU.

    python -m flashfusedmoe_b200.bench_decode [--iters 200] [--warmup 20]
    python -m torch.distributed.run --nproc-per-node N ... -m flashfusedmoe_b200.bench_decode     (expert parallel)

Layer: d_model 7168, 256 routed experts (256 / N per GPU), top-8, swiglu, ffn_dim 2 x 2048, one shared expert of
ffn_dim 2 x 2048, bf16, seed 4, weights N(0, 0.02), 128 tokens per GPU ~ N(0, 1). Every iteration is timed with its
own CUDA-event pair; rank 0 prints one JSON line with p50 / p99 of the per-iteration maximum over ranks, the
all-to-all time measured on the issuing stream, and the weight-streaming bound (local expert bytes / measured HBM
bandwidth) the latency is compared with.
"""

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import MoELayer, ops
from .fused_moe import set_ep_static_forward


def run(iters, warmup, tokens, graph, group, rank, world, dev):
    """Per-iteration latency of the decode-shaped layer on an initialised process group (or one GPU, group None).
    Returns the result dict on rank 0 and None elsewhere."""
    a = argparse.Namespace(iters=iters, warmup=warmup, tokens=tokens, graph=graph)
    D, F, E, k = 7168, 4096, 256, 8
    e_local = E // world
    # build only this rank's experts (the full expert set is 22.5 GB); same seed on every rank for the replicated parts
    torch.manual_seed(4)
    torch.set_default_dtype(torch.bfloat16)  # parameters are created on the GPU in bf16 (no fp32 host copy)
    with torch.device(dev):
        layer = MoELayer(D, F, e_local if world > 1 else E, k, num_shared_experts=1, shared_ffn_dim=F)
        layer.gate = torch.nn.Linear(D, E, bias=False)
    torch.set_default_dtype(torch.float32)
    layer.num_experts = E
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0.0, 0.02)
    if world > 1:
        layer._ep_group = group
        layer._ep_size = world
        from .fused_moe import set_ep_group
        set_ep_group(group)
    torch.manual_seed(4000 + rank)
    x = torch.randn(a.tokens, D, device=dev).bfloat16()
    times = []
    timer = ops.KernelTimer()
    graph = None
    with torch.no_grad():
        if world > 1:
            set_ep_static_forward(a.tokens)   # no host read of the routing counts (eager and captured alike)
        if a.graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    layer(x)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                layer(x)
        for i in range(a.warmup + a.iters):
            if i == a.warmup and graph is None:
                ops.set_timer(timer)
            if world > 1:
                dist.barrier()
            s = torch.cuda.Event(enable_timing=True)
            e = torch.cuda.Event(enable_timing=True)
            s.record()
            if graph is not None:
                graph.replay()
            else:
                layer(x)
            e.record()
            e.synchronize()
            if i >= a.warmup:
                times.append(s.elapsed_time(e))
    ops.set_timer(None)
    ops.check_status()
    if world > 1:
        set_ep_static_forward(None)
    t = torch.tensor(times, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    line = None
    if rank == 0:
        ts = torch.sort(t).values
        kt = timer.totals_ms()
        peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
        hbm = json.load(open(peaks_path))["hbm_gbs"] if os.path.exists(peaks_path) else 6650.0
        weight_bytes = (e_local if world > 1 else E) * (F * D + D * (F // 2)) * 2 + 3 * (F // 2) * D * 2
        line = {"metric": "moe_layer_decode_latency_ms", "unit": "ms", "higher_is_better": False, "n_gpus": world,
                "p50": float(ts[len(ts) // 2]), "p99": float(ts[min(len(ts) - 1, int(len(ts) * 0.99))]),
                "min": float(ts[0]), "iters": a.iters, "tokens_per_gpu": a.tokens, "dtype": "bf16",
                "config": {"workload": "BASELINE configs[4]: d_model=7168 E=256 top_k=8 ffn_dim=4096 + shared expert, forward only",
                           "experts_per_gpu": e_local if world > 1 else E},
                "mode": "cuda graph replay" if a.graph else "eager",
                "weight_stream_bound_ms": weight_bytes / (hbm * 1e9) * 1e3,
                "kernel_ms_per_iter": {n: v[1] / a.iters for n, v in kt.items()}}
        if "all_to_all" in kt:
            line["all_to_all_ms_per_iter"] = kt["all_to_all"][1] / a.iters
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--graph", action="store_true",
                    help="capture the forward pass in a CUDA graph and time replays (expert parallel: uses the "
                         "host-sync-free forward, set_ep_static_forward)")
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
    line = run(a.iters, a.warmup, a.tokens, a.graph, group, rank, world, dev)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
