"""CPU: host-side logic of the package — validation, the reference-compatible helpers, the mock dispatcher and,
over gloo with two ranks, the dispatcher's exchange, expert sharding and the bucketed gradient sync."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import flashfusedmoe_b200 as ffm
from flashfusedmoe_b200.fused_moe import _estimate_max_tokens, _validate_inputs


def test_public_surface():
    for name in ["fused_moe", "set_ep_group", "MoELayer", "ExpertParallelDispatcher",
                 "MockExpertParallelDispatcher", "DispatchHandle", "create_dispatcher", "shard_expert_weights",
                 "OverlappedGradSync", "get_dense_params"]:
        assert hasattr(ffm, name)


def test_estimate_max_tokens_matches_reference_formula():
    # reference tests/test_production.py:37-47
    assert _estimate_max_tokens(1024, 2, 8) == 512
    assert _estimate_max_tokens(4, 2, 8) == 8
    assert _estimate_max_tokens(16384, 2, 8) == 8192
    assert _estimate_max_tokens(100, 6, 64) == 10 + 10


@pytest.mark.parametrize("mutate,msg", [
    (lambda a: a.__setitem__("h", torch.randn(2, 4, 64)), "hidden_states must be 2D"),
    (lambda a: a.__setitem__("g", torch.randn(8, 32)), "gate_weight must be"),
    (lambda a: a.__setitem__("wu", torch.randn(8, 128, 32)), "w_up must be"),
    (lambda a: a.__setitem__("wd", torch.randn(8, 64, 32)), "w_down must be"),
    (lambda a: a.__setitem__("k", 9), "top_k must be in"),
    (lambda a: a.__setitem__("act", "gelu"), "Unknown activation"),
    (lambda a: a.__setitem__("gating", "tanh"), "Unknown gating"),
])
def test_validation_messages(mutate, msg):
    a = dict(h=torch.randn(16, 64), g=torch.randn(8, 64), wu=torch.randn(8, 128, 64), wd=torch.randn(8, 64, 64),
             k=2, act="swiglu", gating="softmax")
    mutate(a)
    with pytest.raises(AssertionError, match=msg):
        _validate_inputs(a["h"], a["g"], a["wu"], a["wd"], a["k"], a["act"], a["gating"])


def test_mock_dispatcher_conservation_and_bytes():
    # reference tests/test_production.py:319-417
    torch.manual_seed(0)
    N, D, E, k, ep = 64, 32, 8, 2, 4
    h = torch.randn(N, D)
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(N)])
    w = torch.rand(N, k)
    mock = ffm.MockExpertParallelDispatcher(E, ep)
    parts = mock.dispatch(h, idx, w)
    assert sum(p[0].shape[0] for p in parts) == N * k
    for rank, (tok, meta) in enumerate(parts):
        assert ((meta["local_expert_ids"] >= 0) & (meta["local_expert_ids"] < E // ep)).all()
    out = mock.combine([p[0] for p in parts], [p[1] for p in parts])
    assert torch.allclose(out, h * k, atol=1e-5)
    stats = mock.get_comm_stats()
    assert stats["dispatch_bytes"] == N * k * D * 4 == stats["combine_bytes"]
    mock.reset_stats()
    assert mock.get_comm_stats()["total_bytes"] == 0


def test_create_dispatcher_backends():
    d = ffm.create_dispatcher(8, 2, None, backend="nccl")
    assert isinstance(d, ffm.ExpertParallelDispatcher) and d.experts_per_gpu == 4
    with pytest.raises(ValueError, match="not available"):
        ffm.create_dispatcher(8, 2, None, backend="deep_ep")
    with pytest.raises(AssertionError, match="divisible"):
        ffm.ExpertParallelDispatcher(7, 2)


def test_get_dense_params_and_layer_state_dict_names():
    layer = ffm.MoELayer(64, 128, 4, 2, num_shared_experts=1, latent_dim=32)
    names = sorted(layer.state_dict().keys())
    assert names == sorted(["gate.weight", "w_up", "w_down", "shared_expert.w_gate.weight",
                            "shared_expert.w_up.weight", "shared_expert.w_down.weight", "proj_down.weight",
                            "proj_up.weight"])
    model = torch.nn.Sequential(torch.nn.Linear(64, 64), layer)
    dense = ffm.get_dense_params(model)
    ids = {id(p) for p in dense}
    assert id(layer.w_up) not in ids and id(layer.w_down) not in ids
    assert id(layer.shared_expert.w_up.weight) in ids and id(layer.gate.weight) in ids
    assert dense[0] is list(model.parameters())[-1]  # backward order


# ---- two gloo ranks ---------------------------------------------------------------------------

def _worker(rank, world, init_file, fn_name, ret):
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    try:
        globals()[fn_name](rank, world)
        ret[rank] = "ok"
    except Exception as e:  # pragma: no cover
        import traceback
        ret[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def _run_two_ranks(fn_name):
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "init")
        mgr = mp.Manager()
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, init_file, fn_name, ret), nprocs=2, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}, dict(ret)


def _case_dispatch_roundtrip(rank, world):
    torch.manual_seed(100 + rank)  # different tokens on every rank
    N, D, E, k = 40 + 8 * rank, 16, 8, 2
    h = torch.randn(N, D)
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(N)])
    disp = ffm.ExpertParallelDispatcher(E, world, None)
    recv, handle = disp.dispatch_fused(h, idx)
    assert recv.shape[0] == sum(handle.recv_splits) == handle.local_expert_ids.numel()
    assert ((handle.local_expert_ids >= 0) & (handle.local_expert_ids < E // world)).all()
    # every rank tags rows with rank-specific values through a fake expert: y = x * (global expert id + 1)
    gid = handle.local_expert_ids + rank * (E // world)
    out = disp.fused_combine(recv * (gid + 1).unsqueeze(-1).to(recv.dtype), handle)
    expect = (h.unsqueeze(1) * (idx + 1).unsqueeze(-1)).reshape(N * k, D)
    assert torch.allclose(out, expect, atol=1e-5)
    # conservation across ranks
    tot = torch.tensor([float(recv.shape[0]), float(N * k)])
    dist.all_reduce(tot)
    assert tot[0] == tot[1]
    # legacy path
    w = torch.rand(N, k)
    recv2, meta = disp.dispatch(h, idx, w)
    out2 = disp.combine(recv2 * meta["received_weights"].unsqueeze(-1), meta)
    assert torch.allclose(out2, h * w.sum(-1, keepdim=True), atol=1e-5)
    # differentiable path: gradient flows back through both exchanges
    hg = h.clone().requires_grad_()
    r3, m3 = disp.dispatch_differentiable(hg, idx, w)
    disp.combine_differentiable(r3 * 2.0, m3).sum().backward()
    assert torch.allclose(hg.grad, torch.full_like(h, 2.0 * k))


def _case_shard_and_gradsync(rank, world):
    torch.manual_seed(0)
    layer = ffm.MoELayer(32, 64, 4, 2, num_shared_experts=1)
    full_up = layer.w_up.data.clone()
    wu, wd = ffm.shard_expert_weights(layer.w_up, layer.w_down, None)
    assert wu.shape[0] == 2 and torch.equal(wu.data, full_up[rank * 2:(rank + 1) * 2])
    dense = ffm.get_dense_params(layer)
    sync = ffm.OverlappedGradSync(dense, dist.group.WORLD, num_buckets=3)
    assert 1 <= sync.num_buckets <= 3 and sum(len(b["params"]) for b in sync.buckets) == len(dense)
    for step in range(2):
        for p in dense:
            p.grad = None
        loss = sum((p * (rank + 1 + step)).sum() for p in dense)
        loss.backward()
        sync.finish()
        for p in dense:
            assert torch.allclose(p.grad, torch.full_like(p, 1.5 + step)), "AVG over ranks 1 and 2 (+step)"
    sync.remove_hooks()
    empty = ffm.OverlappedGradSync([], dist.group.WORLD)
    assert empty.num_buckets == 0
    empty.finish()


def test_dispatcher_roundtrip_gloo():
    _run_two_ranks("_case_dispatch_roundtrip")


def test_shard_and_gradsync_gloo():
    _run_two_ranks("_case_shard_and_gradsync")


def test_segment_plan_moves_every_row_to_the_grouped_layout_and_back():
    """Host tables of the row-granular exchange: simulate all ranks with numpy and check layout, order and padding."""
    import numpy as np
    from flashfusedmoe_b200.p2p import SegmentPlan
    rng = np.random.default_rng(3)
    for ep, e_local in [(2, 4), (4, 2), (8, 1), (4, 16)]:
        E = ep * e_local
        C = rng.integers(0, 700, size=(ep, E))
        C[rng.random((ep, E)) < 0.2] = 0            # some (rank, expert) pairs send nothing
        C[:, 1 % E] = 0                             # one expert receives nothing at all
        plans = [SegmentPlan(C, e_local, r) for r in range(ep)]
        # sender buffers: row id = (source rank, expert, ordinal inside that run)
        send = [[(s, e, j) for e in range(E) for j in range(int(C[s, e]))] for s in range(ep)]
        grouped = [[None] * int(plans[0].rows_grouped[d]) for d in range(ep)]
        for s in range(ep):
            seg, end = plans[s].dispatch
            assert (end[-1] if len(end) else 0) == len(send[s])
            for src0, dst0, rows, d in seg:
                for j in range(rows):
                    assert grouped[d][dst0 + j] is None
                    grouped[d][dst0 + j] = send[s][src0 + j]
        for d in range(ep):
            ts = plans[0].tile_start[d]
            assert (ts % 2 == 0).all() and ts[0] == 0
            for el in range(e_local):
                e = d * e_local + el
                rows = grouped[d][ts[el] * 128:ts[el + 1] * 128]
                valid = [x for x in rows if x is not None]
                assert len(valid) == C[:, e].sum()
                assert rows[:len(valid)] == valid                                  # valid rows first, padding after
                assert valid == sorted(valid) and all(x[1] == e for x in valid)    # source-major, stable inside a source
            seg, _ = plans[d].padding
            padded = sorted(int(dst0 + j) for _, dst0, rows, dd in seg for j in range(rows))
            assert all(dd == d for _, _, _, dd in seg)
            assert padded == [i for i, x in enumerate(grouped[d]) if x is None]
            assert plans[d].recv_rows[d] == sum(x is not None for x in grouped[d])
        # combine direction: every row returns to the position it was sent from
        back = [[None] * len(send[s]) for s in range(ep)]
        for d in range(ep):
            seg, _ = plans[d].combine
            for src0, dst0, rows, s in seg:
                for j in range(rows):
                    back[s][dst0 + j] = grouped[d][src0 + j]
        assert back == send


def test_weight_gradient_split_helpers():
    """Host helpers of the split-K weight gradient: split factor and the tile ranges of the split groups."""
    import sys
    import torch
    import flashfusedmoe_b200  # noqa: F401
    fm = sys.modules["flashfusedmoe_b200.fused_moe"]
    # one expert per rank at D = 1024, H = 2048: dW_down [1024, 2048] has 32 tile pairs -> split in two; dW_up has 64
    assert fm._wgrad_split_factor(1, 1024, 2048) == 2
    assert fm._wgrad_split_factor(1, 4096, 1024) == 1
    assert fm._wgrad_split_factor(8, 1024, 2048) == 1
    assert fm._wgrad_split_factor(4, 256, 256) == 4
    ts = torch.tensor([0, 6, 6, 20, 22], dtype=torch.int32)
    for S in (2, 3, 4):
        cut = fm._split_tile_start(ts, S)
        assert cut.dtype == torch.int32 and cut.numel() == 4 * S + 1
        assert (cut[1:] >= cut[:-1]).all() and (cut % 2 == 0).all()          # whole tile pairs, in order
        assert cut[::S].tolist() == ts.tolist()                               # group boundaries are kept


def test_small_helpers_without_a_gpu():
    import sys
    import torch
    import flashfusedmoe_b200  # noqa: F401
    fm = sys.modules["flashfusedmoe_b200.fused_moe"]
    # run_beside: CPU tensors (or overlap switched off) call the function in place and return no event
    out, ev = fm.run_beside(lambda t: t * 2, torch.ones(3))
    assert ev is None and out.tolist() == [2.0, 2.0, 2.0]
    # side branch for small kernels: none for CPU tensors, and the schedule defaults are on
    assert fm._fork_small(torch.ones(3)) == (None, None)
    assert fm._OVERLAP and fm._FUSED_GLU_BWD
    # inference shortcut arguments of the grouped GEMMs
    assert fm._small_m_kwargs(False, None) == {}
    kw = fm._small_m_kwargs(True, torch.tensor([3, 0, 7], dtype=torch.int64))
    assert kw["tile_rows"] == 128 and kw["valid_rows"].dtype == torch.int32 and kw["valid_rows"].tolist() == [3, 0, 7]
    # the static expert-parallel forward is off unless declared
    assert fm._EP_STATIC_TOKENS is None
    fm.set_ep_static_forward(128)
    assert fm._EP_STATIC_TOKENS == 128
    fm.set_ep_static_forward(None)
    assert fm._EP_STATIC_TOKENS is None


def test_backward_exchanges_alternate_receive_regions():
    """Consecutive backward exchanges of a group must not share a receive region (rows are read in place after the
    barrier while a faster peer may already push the next layer's rows): regions 2 and 3 in turn, per group."""
    import sys
    fm = sys.modules["flashfusedmoe_b200.fused_moe"]
    from flashfusedmoe_b200 import p2p
    assert p2p.NUM_REGIONS == 4
    g1, g2 = object(), object()
    seq1 = [fm._backward_region(g1) for _ in range(5)]
    seq2 = [fm._backward_region(g2) for _ in range(2)]
    assert seq1 == [2, 3, 2, 3, 2] and seq2 == [2, 3]
    assert all(r < p2p.NUM_REGIONS for r in seq1)


def test_expert_gemm_precision_switch():
    import flashfusedmoe_b200 as ffm
    assert ffm.set_expert_gemm_precision("fp8") == "bf16"
    assert ffm.set_expert_gemm_precision("bf16") == "fp8"
    with pytest.raises(ValueError):
        ffm.set_expert_gemm_precision("fp4")
