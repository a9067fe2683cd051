"""Worker for the expert-parallel GPU test: run with torch.distributed.run, one rank per GPU.

Every rank draws different tokens, shards the same full weights, runs the expert-parallel layer and compares with
(a) this package's single-GPU path on the same tokens and full weights, and (b) the CPU oracle for the pieces the
single-GPU path cannot express (routing-only input gradient, latent projection). Exit code 0 means every check
passed on every rank.
"""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import flashfusedmoe_b200 as ffm  # noqa: E402
from flashfusedmoe_b200 import ops  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

TOL = 2e-2


def rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda")
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    group = dist.group.WORLD

    N, D, E, F, k = 384 + 64 * rank, 256, 8, 512, 2
    H = F // 2
    torch.manual_seed(7)  # weights: same on every rank
    g = (torch.randn(E, D) * 0.05).bfloat16().to(dev)
    wu = (torch.randn(E, F, D) * 0.05).bfloat16().to(dev)
    wd = (torch.randn(E, D, H) * 0.05).bfloat16().to(dev)
    sg, su = [(torch.randn(H, D) * 0.05).bfloat16().to(dev) for _ in range(2)]
    sd = (torch.randn(D, H) * 0.05).bfloat16().to(dev)
    L = 128
    lwd = (torch.randn(L, D) * 0.06).bfloat16().to(dev)
    lwu = (torch.randn(D, L) * 0.09).bfloat16().to(dev)
    torch.manual_seed(100 + rank)  # tokens: different on every rank
    h = torch.randn(N, D).bfloat16().to(dev)
    go = torch.randn(N, D).bfloat16().to(dev)
    El = E // world
    wu_l = wu[rank * El:(rank + 1) * El].clone()
    wd_l = wd[rank * El:(rank + 1) * El].clone()

    # ---- plain EP vs single GPU ------------------------------------------------------------
    hp, gp, wup, wdp = [t.clone().requires_grad_() for t in (h, g, wu_l, wd_l)]
    out_ep, losses = ffm.fused_moe(hp, gp, wup, wdp, top_k=k, ep_group=group, aux_loss_coeff=0.01, return_metrics=True)
    (out_ep.float() * go.float()).sum().backward()
    ops.check_status()
    hs, gs, wus, wds = [t.clone().requires_grad_() for t in (h, g, wu, wd)]
    out_1, losses_1 = ffm.fused_moe(hs, gs, wus, wds, top_k=k, aux_loss_coeff=0.01, return_metrics=True)
    (out_1.float() * go.float()).sum().backward()
    assert torch.equal(losses["tokens_per_expert"], losses_1["tokens_per_expert"])
    assert rel(out_ep, out_1) <= 1e-6, f"EP output differs from single GPU: {rel(out_ep, out_1)}"
    # the other transport gives bit-identical results
    fm = sys.modules["flashfusedmoe_b200.fused_moe"]  # the package rebinds the name fused_moe to the function
    this_transport = fm._EP_TRANSPORT
    fm._EP_TRANSPORT = "nccl" if this_transport == "p2p" else "p2p"
    ho, go_, wuo, wdo = [t.clone().requires_grad_() for t in (h, g, wu_l, wd_l)]
    out_o, _ = ffm.fused_moe(ho, go_, wuo, wdo, top_k=k, ep_group=group, aux_loss_coeff=0.01)
    (out_o.float() * go.float()).sum().backward()
    fm._EP_TRANSPORT = this_transport
    assert torch.equal(out_o, out_ep) and torch.equal(wuo.grad, wup.grad) and torch.equal(ho.grad, hp.grad), \
        "p2p and nccl transports must agree bit for bit"
    assert rel(gp.grad, gs.grad) <= 1e-3, "gate gradient"
    assert abs(float(losses["aux_loss"]) - float(losses_1["aux_loss"])) < 1e-6
    # expert weight gradients: sum over all ranks' tokens, scaled by 1 / ep (reference: fused_moe.py:961-966)
    full_wu, full_wd = wus.grad.float().clone(), wds.grad.float().clone()
    dist.all_reduce(full_wu)
    dist.all_reduce(full_wd)
    assert rel(wup.grad, full_wu[rank * El:(rank + 1) * El] / world) <= TOL, "dW_up"
    assert rel(wdp.grad, full_wd[rank * El:(rank + 1) * El] / world) <= TOL, "dW_down"
    # input gradient holds the routing term only (reference: fused_moe.py:1001-1005)
    fw = orc.fused_moe_forward(h.cpu(), g.cpu(), wu.cpu(), wd.cpu(), k, dtype=torch.bfloat16)
    bw = orc.fused_moe_backward(fw, go.cpu())
    route_only = orc.mm(bw["gl"], g.cpu(), torch.bfloat16)
    assert rel(hp.grad, route_only) <= 5e-2, f"routing-only dH {rel(hp.grad, route_only)}"

    # opt-in complete input gradient: equals the single-GPU dH
    hf = h.clone().requires_grad_()
    out_f, _ = ffm.fused_moe(hf, g, wu_l, wd_l, top_k=k, ep_group=group, ep_full_input_grad=True)
    (out_f.float() * go.float()).sum().backward()
    hs2 = h.clone().requires_grad_()
    out_2, _ = ffm.fused_moe(hs2, g, wu, wd, top_k=k)
    (out_2.float() * go.float()).sum().backward()
    assert rel(hf.grad, hs2.grad) <= TOL, f"full EP input gradient {rel(hf.grad, hs2.grad)}"

    # ---- shared expert inside the EP call ----------------------------------------------------
    hq = h.clone().requires_grad_()
    sgp, sup, sdp = [t.clone().requires_grad_() for t in (sg, su, sd)]
    out_s, _ = ffm.fused_moe(hq, g, wu_l, wd_l, top_k=k, ep_group=group, shared_expert_weights=(sgp, sup, sdp))
    (out_s.float() * go.float()).sum().backward()
    shared = orc.glu_ffn(h.cpu(), sg.cpu(), su.cpu(), sd.cpu(), "swiglu", torch.bfloat16)
    assert rel(out_s, out_1.detach().float().cpu() + shared.float()) <= TOL, "shared expert output"
    xs = h.cpu().float().requires_grad_()
    ws = [t.cpu().float().requires_grad_() for t in (sg, su, sd)]
    ((torch.nn.functional.silu(xs @ ws[0].T) * (xs @ ws[1].T)) @ ws[2].T * go.cpu().float()).sum().backward()
    for name, ours, ref in zip(("w_gate", "w_up", "w_down"), (sgp, sup, sdp), ws):
        assert rel(ours.grad, ref.grad) <= TOL, f"shared {name} gradient"
    assert rel(hq.grad, route_only.float() + xs.grad) <= 5e-2, "dH with shared expert"

    # ---- latent projection around both exchanges ---------------------------------------------
    lwdp, lwup = lwd.clone().requires_grad_(), lwu.clone().requires_grad_()
    wul, wdl = wu_l.clone().requires_grad_(), wd_l.clone().requires_grad_()
    out_l, _ = ffm.fused_moe(h, g, wul, wdl, top_k=k, ep_group=group, latent_weights=(lwdp, lwup))
    (out_l.float() * go.float()).sum().backward()
    ops.check_status()
    bf = torch.bfloat16
    hc, gc = h.cpu(), g.cpu()
    x2 = orc.mm(orc.mm(hc, lwd.cpu().T, bf), lwu.cpu().T, bf)  # project down, exchange, project up
    w, idx = orc.route(orc.gate_logits(hc, gc, bf), "softmax", k)
    ref = torch.zeros(N, D)
    for j in range(k):
        for e in range(E):
            m = idx[:, j] == e
            if m.any():
                pre = orc.mm(x2[m], wu.cpu()[e].T, bf)
                y = orc.mm(orc.glu_forward(pre, "swiglu", bf), wd.cpu()[e].T, bf)
                y = orc.mm(orc.mm(y, lwd.cpu().T, bf), lwu.cpu().T, bf)
                ref[m] += w[m, j].to(bf).float().unsqueeze(-1) * y.float()
    assert rel(out_l, ref) <= TOL, f"latent output {rel(out_l, ref)}"
    for t in (lwdp.grad, lwup.grad, wul.grad, wdl.grad):
        assert t is not None and torch.isfinite(t).all()
    hl = h.clone().requires_grad_()
    out_lf, _ = ffm.fused_moe(hl, g, wu_l, wd_l, top_k=k, ep_group=group, latent_weights=(lwd, lwu),
                              ep_full_input_grad=True)
    (out_lf.float() * go.float()).sum().backward()
    assert torch.equal(out_lf, out_l.detach()) and torch.isfinite(hl.grad).all()
    assert (hl.grad.float() - route_only.to(dev).float()).abs().max() > 0, "latent path adds the expert input gradient"

    # ---- host-sync-free forward (inference), eager and replayed from a CUDA graph ---------------------------------
    if fm._EP_TRANSPORT == "p2p":
        with torch.no_grad():
            ref_out, ref_losses = ffm.fused_moe(h, g, wu_l, wd_l, top_k=k, ep_group=group,
                                                shared_expert_weights=(sg, su, sd), return_metrics=True)
            ffm.set_ep_static_forward(384 + 64 * world)    # the same bound on every rank (ranks hold different N)
            st_out, st_losses = ffm.fused_moe(h, g, wu_l, wd_l, top_k=k, ep_group=group,
                                              shared_expert_weights=(sg, su, sd), return_metrics=True)
            ops.check_status()
            assert torch.equal(st_out, ref_out), f"static forward differs: {rel(st_out, ref_out)}"
            assert torch.equal(st_losses["tokens_per_expert"], ref_losses["tokens_per_expert"])
            # graph: capture once, replay on new tokens
            h_static = h.clone()
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(2):
                    ffm.fused_moe(h_static, g, wu_l, wd_l, top_k=k, ep_group=group, shared_expert_weights=(sg, su, sd))
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                g_out, _ = ffm.fused_moe(h_static, g, wu_l, wd_l, top_k=k, ep_group=group,
                                         shared_expert_weights=(sg, su, sd))
            torch.manual_seed(500 + rank)
            h_new = torch.randn(N, D).bfloat16().to(dev)
            for src in (h, h_new, h):
                h_static.copy_(src)
                graph.replay()
                torch.cuda.synchronize()
                ffm.set_ep_static_forward(None)
                want, _ = ffm.fused_moe(src, g, wu_l, wd_l, top_k=k, ep_group=group, shared_expert_weights=(sg, su, sd))
                ffm.set_ep_static_forward(384 + 64 * world)
                assert torch.equal(g_out, want), f"graph replay differs: {rel(g_out, want)}"
            ops.check_status()
            ffm.set_ep_static_forward(None)

    # ---- MoELayer.shard_experts ----------------------------------------------------------------
    torch.manual_seed(3)
    layer = ffm.MoELayer(D, F, E, k, num_shared_experts=1).to(dev).bfloat16()
    layer.shard_experts(group)
    assert layer.w_up.shape[0] == El
    y, _ = layer(h.view(1, N, D))
    y.float().sum().backward()
    assert torch.isfinite(y).all() and layer.w_up.grad is not None
    dense = ffm.get_dense_params(layer)
    sync = ffm.OverlappedGradSync(dense, group, num_buckets=2)
    for p in layer.parameters():
        p.grad = None
    y, _ = layer(h.view(1, N, D))
    y.float().sum().backward()
    sync.finish()
    gsum = layer.gate.weight.grad.float().clone()
    chk = gsum.clone()
    dist.all_reduce(chk)
    assert rel(chk / world, gsum) <= 1e-6, "dense gradients are averaged across ranks"
    ffm.set_ep_group(None)
    ops.check_status()
    torch.cuda.synchronize()
    dist.barrier()
    print(f"EP_OK rank {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
