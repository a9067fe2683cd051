"""Expert-parallel token dispatch / combine over torch.distributed.

Host-side plumbing with the interface of the reference's dispatcher classes
(src/flashfusemoe/expert_parallel.py:56-64 DispatchHandle, :94-433 ExpertParallelDispatcher,
:436-563 MockExpertParallelDispatcher, :660-688 create_dispatcher). The arithmetic of the layer does not live
here: these classes only move rows between ranks, with torch index ops and c10d collectives, so they run on
any device c10d supports (NCCL on GPUs, gloo in the CPU tests).

Differences from the reference, all internal to the exchange:
  * rows are ordered by (destination rank, expert, token) instead of (destination rank, token), so the
    receiver can rebuild the expert id of every row from the exchanged [ep, E_local] count matrix and no
    id column travels with the payload (the reference appends the id as one extra bf16 element per row,
    fused_dispatch.py:20-66);
  * one host synchronisation per dispatch, on a single [2, ep] tensor, instead of two pinned copies.
"""

from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class DispatchHandle:
    """Metadata from dispatch needed for combine (reference: expert_parallel.py:56-64)."""
    sort_order: torch.Tensor        # [N*top_k] flat slots in send order
    send_splits: list               # rows sent to each EP rank
    recv_splits: list               # rows received from each EP rank
    N: int
    top_k: int
    local_expert_ids: torch.Tensor  # [M] local expert of every received row
    recv_counts: torch.Tensor = field(default=None, repr=False)  # [ep, E_local] rows per (source, local expert)


class _AllToAllAutograd(torch.autograd.Function):
    """Differentiable variable-split all-to-all; backward is the reverse exchange
    (reference: expert_parallel.py:67-91)."""

    @staticmethod
    def forward(ctx, input_tensor, output_split_sizes, input_split_sizes, group):
        ctx.output_split_sizes = output_split_sizes
        ctx.input_split_sizes = input_split_sizes
        ctx.group = group
        return all_to_all_rows(input_tensor.contiguous(), output_split_sizes, input_split_sizes, group)

    @staticmethod
    def backward(ctx, grad_output):
        grad_input = all_to_all_rows(grad_output.contiguous(), ctx.input_split_sizes, ctx.output_split_sizes,
                                     ctx.group)
        return grad_input, None, None, None


def all_to_all_rows(rows, out_splits, in_splits, group):
    """Variable-split all-to-all over the leading dimension; returns a fresh tensor."""
    out = rows.new_empty((int(sum(out_splits)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows, list(out_splits), list(in_splits), group=group)
    return out


def exchange_counts(per_expert_counts, ep_size, group):
    """All-to-all of the [ep, E_local] per-expert row counts.

    Returns (recv_counts [ep, E_local] on the device, send_splits, recv_splits as python lists).
    The single `.tolist()` here is the only host synchronisation of a dispatch.
    """
    send_mat = per_expert_counts.reshape(ep_size, -1).to(torch.int64).contiguous()
    recv_mat = torch.empty_like(send_mat)
    dist.all_to_all_single(recv_mat, send_mat, group=group)
    both = torch.stack([send_mat.sum(1), recv_mat.sum(1)]).tolist()
    return recv_mat, [int(v) for v in both[0]], [int(v) for v in both[1]]


def local_ids_from_counts(recv_counts, total_rows):
    """Expert id of every received row, from the [ep, E_local] count matrix (rows arrive source-major,
    expert-minor)."""
    ep, e_local = recv_counts.shape
    ids = torch.arange(e_local, device=recv_counts.device).repeat(ep)
    return torch.repeat_interleave(ids, recv_counts.reshape(-1), output_size=int(total_rows))


class ExpertParallelDispatcher:
    """Dispatches token rows to expert-owning ranks via all-to-all (reference: expert_parallel.py:94-433)."""

    def __init__(self, num_experts, ep_size, process_group=None):
        assert num_experts % ep_size == 0, \
            f"num_experts ({num_experts}) must be divisible by ep_size ({ep_size})"
        self.num_experts = num_experts
        self.ep_size = ep_size
        self.experts_per_gpu = num_experts // ep_size
        self.process_group = process_group

    def _get_group(self):
        return self.process_group if self.process_group is not None else dist.group.WORLD

    # -- fused path ---------------------------------------------------------------------------
    def dispatch_fused(self, hidden_states, topk_indices):
        """hidden_states [N, D], topk_indices [N, top_k] -> (received rows [M, D], DispatchHandle)."""
        N, D = hidden_states.shape
        top_k = topk_indices.shape[1]
        group = self._get_group()
        flat = topk_indices.reshape(-1).to(torch.int64)
        counts = torch.bincount(flat, minlength=self.num_experts)
        recv_counts, send_splits, recv_splits = exchange_counts(counts, self.ep_size, group)
        sort_order = torch.argsort(flat, stable=True)  # expert-major == destination-major
        send = hidden_states[sort_order // top_k]
        received = all_to_all_rows(send, recv_splits, send_splits, group)
        local_ids = local_ids_from_counts(recv_counts, sum(recv_splits))
        handle = DispatchHandle(sort_order=sort_order, send_splits=send_splits, recv_splits=recv_splits, N=N,
                                top_k=top_k, local_expert_ids=local_ids, recv_counts=recv_counts)
        return received, handle

    def fused_combine(self, expert_outputs, handle):
        """expert_outputs [M, D] -> [N*top_k, D] in flat slot order (caller applies weights and sums)."""
        group = self._get_group()
        returned = all_to_all_rows(expert_outputs.contiguous(), handle.send_splits, handle.recv_splits, group)
        unsorted = torch.empty_like(returned)
        unsorted[handle.sort_order] = returned
        return unsorted

    # -- legacy three-tensor path (reference: expert_parallel.py:123-193, :300-433) ------------
    def _dispatch_impl(self, hidden_states, topk_indices, topk_weights, differentiable):
        N, D = hidden_states.shape
        top_k = topk_indices.shape[1]
        group = self._get_group()
        rank = dist.get_rank(group)
        flat = topk_indices.reshape(-1).to(torch.int64)
        counts = torch.bincount(flat, minlength=self.num_experts)
        recv_counts, send_splits, recv_splits = exchange_counts(counts, self.ep_size, group)
        sort_order = torch.argsort(flat, stable=True)
        sorted_hidden = hidden_states[sort_order // top_k]
        if differentiable:
            received = _AllToAllAutograd.apply(sorted_hidden, recv_splits, send_splits, group)
        else:
            received = all_to_all_rows(sorted_hidden, recv_splits, send_splits, group)
        received_weights = all_to_all_rows(topk_weights.reshape(-1)[sort_order].contiguous(), recv_splits,
                                           send_splits, group)
        local_ids = local_ids_from_counts(recv_counts, sum(recv_splits))
        metadata = {
            "sort_order": sort_order,
            "send_counts": torch.tensor(send_splits, device=hidden_states.device),
            "recv_counts": torch.tensor(recv_splits, device=hidden_states.device),
            "send_splits": send_splits,
            "recv_splits": recv_splits,
            "N": N,
            "top_k": top_k,
            "local_expert_ids": local_ids,
            "received_weights": received_weights,
            "rank": rank,
        }
        return received, metadata

    def dispatch(self, hidden_states, topk_indices, topk_weights):
        return self._dispatch_impl(hidden_states, topk_indices, topk_weights, differentiable=False)

    def dispatch_differentiable(self, hidden_states, topk_indices, topk_weights):
        return self._dispatch_impl(hidden_states, topk_indices, topk_weights, differentiable=True)

    def _combine_impl(self, expert_outputs, metadata, differentiable):
        group = self._get_group()
        send_splits, recv_splits = metadata["recv_splits"], metadata["send_splits"]
        if differentiable:
            returned = _AllToAllAutograd.apply(expert_outputs, recv_splits, send_splits, group)
        else:
            returned = all_to_all_rows(expert_outputs.contiguous(), recv_splits, send_splits, group)
        inv = torch.empty_like(metadata["sort_order"])
        inv[metadata["sort_order"]] = torch.arange(inv.numel(), device=inv.device)
        unsorted = returned[inv]
        return unsorted.view(metadata["N"], metadata["top_k"], returned.shape[-1]).sum(dim=1)

    def combine(self, expert_outputs, metadata):
        return self._combine_impl(expert_outputs, metadata, differentiable=False)

    def combine_differentiable(self, expert_outputs, metadata):
        return self._combine_impl(expert_outputs, metadata, differentiable=True)


class MockExpertParallelDispatcher:
    """Single-process stand-in that partitions rows as EP would and counts the bytes that would cross ranks
    (reference: expert_parallel.py:436-563)."""

    def __init__(self, num_experts, ep_size):
        assert num_experts % ep_size == 0, \
            f"num_experts ({num_experts}) must be divisible by ep_size ({ep_size})"
        self.num_experts = num_experts
        self.ep_size = ep_size
        self.experts_per_gpu = num_experts // ep_size
        self.reset_stats()

    def reset_stats(self):
        self.dispatch_bytes = 0
        self.combine_bytes = 0
        self.total_dispatch_tokens = 0
        self.total_combine_tokens = 0

    def dispatch(self, hidden_states, topk_indices, topk_weights):
        N, D = hidden_states.shape
        top_k = topk_indices.shape[1]
        flat_idx = topk_indices.reshape(-1)
        flat_w = topk_weights.reshape(-1)
        dest = flat_idx // self.experts_per_gpu
        expanded = hidden_states.unsqueeze(1).expand(-1, top_k, -1).reshape(N * top_k, D)
        results = []
        for rank in range(self.ep_size):
            mask = dest == rank
            count = int(mask.sum().item())
            self.dispatch_bytes += count * D * hidden_states.element_size()
            self.total_dispatch_tokens += count
            metadata = {"mask": mask, "N": N, "top_k": top_k, "D": D, "rank": rank,
                        "local_expert_ids": flat_idx[mask] - rank * self.experts_per_gpu,
                        "received_weights": flat_w[mask], "count": count}
            results.append((expanded[mask], metadata))
        return results

    def combine(self, all_expert_outputs, all_metadata):
        meta0 = all_metadata[0]
        N, top_k, D = meta0["N"], meta0["top_k"], meta0["D"]
        first = all_expert_outputs[0]
        flat = torch.zeros(N * top_k, D, dtype=first.dtype, device=first.device)
        for rank in range(self.ep_size):
            count = all_metadata[rank]["count"]
            self.combine_bytes += count * D * first.element_size()
            self.total_combine_tokens += count
            flat[all_metadata[rank]["mask"]] = all_expert_outputs[rank]
        return flat.view(N, top_k, D).sum(dim=1)

    def get_comm_stats(self):
        return {"dispatch_bytes": self.dispatch_bytes, "combine_bytes": self.combine_bytes,
                "total_bytes": self.dispatch_bytes + self.combine_bytes,
                "dispatch_tokens": self.total_dispatch_tokens, "combine_tokens": self.total_combine_tokens}


def create_dispatcher(num_experts, ep_size, process_group=None, backend="nccl", **kwargs):
    """Factory (reference: expert_parallel.py:660-688). Only the c10d all-to-all backend exists here;
    the reference's optional DeepEP / hybrid backends wrap an external NVSHMEM library and are refused."""
    if backend != "nccl":
        raise ValueError(
            f"ep backend {backend!r} is not available: this package ships one expert-parallel transport "
            "(torch.distributed all-to-all over NVLink); use backend='nccl'")
    return ExpertParallelDispatcher(num_experts, ep_size, process_group)
