"""Expert-parallel utilities: weight sharding and dense-gradient all-reduce overlapped with backward
(reference: src/flashfusemoe/distributed.py:12-206). Pure torch / torch.distributed host code; runs on any
device c10d supports."""

import torch
import torch.distributed as dist
import torch.nn as nn


def shard_expert_weights(w_up, w_down, ep_group):
    """Slice [E, ...] expert weights to this rank's contiguous block of E / ep_size experts
    (reference: distributed.py:12-33). Returns new nn.Parameters."""
    rank = dist.get_rank(ep_group)
    ep_size = dist.get_world_size(ep_group)
    E = w_up.shape[0]
    assert E % ep_size == 0, f"n_experts ({E}) must be divisible by ep_size ({ep_size})"
    e_local = E // ep_size
    lo, hi = rank * e_local, (rank + 1) * e_local
    return nn.Parameter(w_up.data[lo:hi].contiguous()), nn.Parameter(w_down.data[lo:hi].contiguous())


def get_dense_params(model, backward_order=True):
    """Parameters replicated on every EP rank, i.e. everything but the routed experts
    (reference: distributed.py:36-79). With backward_order the list is reversed (last layer first)."""
    from .nn import MoELayer

    expert_ids = set()
    for m in model.modules():
        if isinstance(m, MoELayer):
            expert_ids.update(id(p) for p in m.expert_params)
    if not expert_ids:
        for name, p in model.named_parameters():
            if ("w_up" in name or "w_down" in name) and "shared_expert" not in name:
                expert_ids.add(id(p))
    dense, seen = [], set()
    for _name, p in model.named_parameters():
        if not p.requires_grad or id(p) in seen:
            continue
        seen.add(id(p))
        if id(p) not in expert_ids:
            dense.append(p)
    return list(reversed(dense)) if backward_order else dense


class OverlappedGradSync:
    """Bucketed AVG all-reduce of dense gradients, fired from post-accumulate-grad hooks while backward is still
    running; `finish()` waits and copies the averaged values back (reference: distributed.py:82-206).

    Buckets hold roughly equal element counts in the given (backward) order. On CUDA each bucket's all-reduce
    runs on a side stream fenced with events; on CPU (gloo) it runs inline. Buckets are packed and unpacked with
    one fused torch._foreach copy instead of a Python loop of slice copies.
    """

    def __init__(self, params, process_group, num_buckets=4):
        self.process_group = process_group
        self.num_buckets = num_buckets
        self._hooks = []
        self.buckets = []
        params = list(params)
        if not params:
            self.num_buckets = 0
            return
        total = sum(p.numel() for p in params)
        target = total / num_buckets
        cur, cur_n = [], 0
        for p in params:
            cur.append(p)
            cur_n += p.numel()
            if cur_n >= target and len(self.buckets) < num_buckets - 1:
                self.buckets.append(self._make_bucket(cur))
                cur, cur_n = [], 0
        if cur:
            self.buckets.append(self._make_bucket(cur))
        self.num_buckets = len(self.buckets)
        device = params[0].device
        self._cuda = device.type == "cuda"
        self._comm_stream = torch.cuda.Stream(device=device) if self._cuda else None
        for bi, bucket in enumerate(self.buckets):
            for p in bucket["params"]:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(bi)))

    @staticmethod
    def _make_bucket(params):
        total = sum(p.numel() for p in params)
        flat = torch.empty(total, dtype=params[0].dtype, device=params[0].device)
        views, off = [], 0
        for p in params:
            views.append(flat[off:off + p.numel()].view(p.shape))
            off += p.numel()
        return {"params": list(params), "flat": flat, "views": views, "count": 0, "expected": len(params),
                "done_event": None}

    def _launch(self, bucket):
        torch._foreach_copy_(bucket["views"], [p.grad for p in bucket["params"]])
        if not self._cuda:
            dist.all_reduce(bucket["flat"], op=dist.ReduceOp.SUM, group=self.process_group)
            bucket["flat"].div_(dist.get_world_size(self.process_group))
            bucket["done_event"] = True
            return
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ready)
            dist.all_reduce(bucket["flat"], op=dist.ReduceOp.AVG, group=self.process_group)
            ev = torch.cuda.Event()
            ev.record()
        bucket["done_event"] = ev

    def _make_hook(self, bucket_idx):
        def hook(_param):
            bucket = self.buckets[bucket_idx]
            bucket["count"] += 1
            if bucket["count"] == bucket["expected"]:
                self._launch(bucket)
        return hook

    def finish(self):
        """Call right after loss.backward(): waits for every bucket and writes the averages into .grad."""
        if self.num_buckets == 0:
            return
        for bucket in self.buckets:
            if bucket["done_event"] is None:
                continue
            if self._cuda:
                torch.cuda.current_stream().wait_event(bucket["done_event"])
            torch._foreach_copy_([p.grad for p in bucket["params"]], bucket["views"])
        for bucket in self.buckets:
            bucket["count"] = 0
            bucket["done_event"] = None

    def remove_hooks(self):
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
