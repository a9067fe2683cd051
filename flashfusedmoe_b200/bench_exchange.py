"""Bandwidth of the expert-parallel row exchange alone (no layer around it), one process per GPU.

    python -m torch.distributed.run --nproc-per-node N ... -m flashfusedmoe_b200.bench_exchange [--rows 32768] [--width 1024]

Every rank holds `rows` bf16 rows of `width` columns sorted by expert (uniform counts over E = 8 * N experts) and
pushes them into the owners' grouped layouts with ffm_p2p_push_rows, then joins the flag barrier. Timed with CUDA
events on the issuing stream, after a group barrier, maximum over ranks:
  push      the store kernel alone (bytes that leave the GPU / time = NVLink GB/s per direction)
  exchange  push + flag barrier (what a layer waits for)
and the same for the NCCL all_to_all_single of the same rows. Rank 0 prints one JSON line.
"""

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from . import ops, p2p


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=50)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    e_local = 8
    E = e_local * world
    per = a.rows // E
    C = np.full((world, E), per, dtype=np.int64)
    sp = p2p.SegmentPlan(C, e_local, rank)
    rb = a.width * 2
    px = p2p.get_exchange(group, dev, int(sp.rows_grouped.max()) * rb)
    seg, end = px.upload(sp.dispatch[0], sp.dispatch[1])
    rows = torch.randn(per * E, a.width, device=dev).bfloat16()
    remote_rows = int(sp.dispatch[0][sp.dispatch[0][:, 3] != rank, 2].sum())
    total = per * E

    def timed(fn_push, fn_rest):
        push_ms, all_ms = [], []
        for i in range(a.iters + 5):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            fn_push()
            e1.record()
            fn_rest()
            e2.record()
            torch.cuda.synchronize()
            if i >= 5:
                push_ms.append(e0.elapsed_time(e1))
                all_ms.append(e0.elapsed_time(e2))
        t = torch.tensor([np.median(push_ms), np.median(all_ms)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]), float(t[1])

    p_push, p_all = timed(lambda: px.push_rows(rows, None, 1, rb, seg, end, len(sp.dispatch[0]), total, 0),
                          lambda: px.barrier())
    out = torch.empty_like(rows)
    splits = [per * e_local] * world
    n_push, n_all = timed(lambda: dist.all_to_all_single(out, rows, splits, splits, group=group), lambda: None)
    ops.check_status()
    if rank == 0:
        gb = remote_rows * rb / 1e9
        print(json.dumps({"metric": "ep_exchange_bandwidth", "n_gpus": world, "rows": total, "row_bytes": rb,
                          "bytes_leaving_per_gpu": remote_rows * rb,
                          "peer_store_push_ms": p_push, "peer_store_push_gbs_per_direction": gb / (p_push * 1e-3),
                          "peer_store_exchange_ms": p_all, "peer_store_exchange_gbs": gb / (p_all * 1e-3),
                          "nccl_all_to_all_ms": n_all, "nccl_gbs": gb / (n_all * 1e-3),
                          "frac_of_770_push": gb / (p_push * 1e-3) / 770.0}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
