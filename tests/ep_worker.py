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


def tokens_of(rank_s, D):
    """The tokens and output gradient rank `rank_s` draws (CPU generator, so every rank can regenerate them)."""
    torch.manual_seed(100 + rank_s)
    n = 384 + 64 * rank_s
    return torch.randn(n, D).bfloat16(), torch.randn(n, D).bfloat16()


def latent_reference(rank, world, D, E, k, g, wu, wd, lwd, lwu, dev):
    """fp32 simulation of the whole group for the latent-projection layer. Returns what rank `rank` must hold:
    d proj_up = (grad_flat^T unsorted_latent [own tokens] + recv_grad_D^T received_latent [rows it owns]) / ep,
    d proj_down = recv_grad_latent^T local_out_D / ep (reference fused_moe.py:988-999), and the expert weight
    gradients of every expert scaled by 1 / ep (:961-966)."""
    F = torch.nn.functional
    El = E // world
    H = wu.shape[1] // 2
    gf, wuf, wdf, lwdf, lwuf = (t.float() for t in (g, wu, wd, lwd, lwu))
    d_lwu = torch.zeros_like(lwuf)
    d_lwd = torch.zeros_like(lwdf)
    d_wu = torch.zeros_like(wuf)
    d_wd = torch.zeros_like(wdf)
    for s in range(world):
        h_s, go_s = (t.to(dev) for t in tokens_of(s, D))
        r = ops.route_forward(h_s, g, k, "softmax")
        idx = r.topk_idx.long()
        wts = torch.softmax(r.logits.float().gather(1, idx), -1).bfloat16().float()
        z = h_s.float() @ lwdf.T                      # dispatch projection [n, L]
        x2 = z @ lwuf.T                               # un-projection at the owner [n, D]
        for e in range(E):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            pre = x2[tok] @ wuf[e].T
            gate, up = pre[:, :H], pre[:, H:]
            sg = torch.sigmoid(gate)
            a = gate * sg * up
            y = a @ wdf[e].T                          # local_out_D
            ul = y @ lwdf.T                           # unsorted_latent, back at the sender
            gflat = go_s[tok].float() * wts[tok, slot].unsqueeze(1)
            gfl = gflat @ lwuf                        # travels to the owner: recv_grad_latent
            rgd = gfl @ lwuf.T                        # recv_grad in D
            if s == rank:
                d_lwu += gflat.T @ ul
            if e // El == rank:
                d_lwu += rgd.T @ z[tok]
                d_lwd += gfl.T @ y
            d_wd[e] += rgd.T @ a
            da = rgd @ wdf[e]
            gu = torch.cat([da * up * (sg * (1 + gate * (1 - sg))), da * gate * sg], 1)
            d_wu[e] += gu.T @ x2[tok]
    return d_lwu / world, d_lwd / world, d_wu / world, d_wd / world


def two_layer_stack(x, layers, k, group, bias, latent, full_grad, between=None):
    """Two expert-parallel layers back to back (residual in between), the shape of a model whose backward issues
    one exchange per layer with nothing but compute between them. `between` runs when the gradient of the
    intermediate activation is ready, i.e. between the two layers' backward passes."""
    h = x
    for i, (gw, wu, wd, lw) in enumerate(layers):
        y, _ = ffm.fused_moe(h, gw, wu, wd, top_k=k, ep_group=group, expert_bias=bias,
                             latent_weights=lw if latent else None, ep_full_input_grad=full_grad)
        h = h + y
        if i == 0 and between is not None:
            h.register_hook(lambda grad: (between(), grad)[1])
    return h


def stacked_layers_case(rank, world, group, dev):
    """Skewed routing (a gate bias sends most rows to the experts of the last rank) so that ranks finish a layer's
    backward at very different times, two layers, several steps. The gradients must be bit-identical to a run that
    puts a device synchronisation and a group barrier between the two layers' backward passes (no rank can then run
    ahead into the next exchange), and, without latent projection and with the complete input gradient, agree with
    the single-GPU path on the full weights."""
    N, D, E, F, k, L = 4096 + 256 * rank, 512, 8, 1024, 2, 128
    El = E // world
    torch.manual_seed(21)
    full = []
    for _ in range(2):
        full.append(((torch.randn(E, D) * 0.05).bfloat16().to(dev), (torch.randn(E, F, D) * 0.05).bfloat16().to(dev),
                     (torch.randn(E, D, F // 2) * 0.05).bfloat16().to(dev),
                     ((torch.randn(L, D) * 0.06).bfloat16().to(dev), (torch.randn(D, L) * 0.09).bfloat16().to(dev))))
    bias = torch.zeros(E, device=dev)
    bias[E - El:] = 1.5                                 # most rows go to the last rank's experts
    torch.manual_seed(300 + rank)
    x = torch.randn(N, D).bfloat16().to(dev)
    go = torch.randn(N, D).bfloat16().to(dev)

    def barrier_between():
        torch.cuda.synchronize()
        dist.barrier()

    def run(latent, full_grad, between, steps=3):
        grads = None
        for _ in range(steps):
            layers = [(gw.clone().requires_grad_(), wu[rank * El:(rank + 1) * El].clone().requires_grad_(),
                       wd[rank * El:(rank + 1) * El].clone().requires_grad_(),
                       tuple(t.clone().requires_grad_() for t in lw)) for gw, wu, wd, lw in full]
            xin = x.clone().requires_grad_()
            out = two_layer_stack(xin, layers, k, group, bias, latent, full_grad, between)
            (out.float() * go.float()).sum().backward()
            grads = [xin.grad] + [t.grad for lay in layers for t in (lay[0], lay[1], lay[2])]
            if latent:
                grads += [t.grad for lay in layers for t in lay[3]]
        ops.check_status()
        return out.detach(), grads

    for latent, full_grad in ((False, True), (True, False), (True, True)):
        out_a, grads_a = run(latent, full_grad, None)
        out_b, grads_b = run(latent, full_grad, barrier_between)
        assert torch.equal(out_a, out_b)
        for i, (a, b) in enumerate(zip(grads_a, grads_b)):
            assert torch.equal(a, b), f"gradient {i} changes when the ranks are kept in step (latent={latent})"
        if not latent:
            # the host-sync-free path gives the same two-layer results, with and without the ranks kept in step
            ffm.set_ep_static_forward(4096 + 256 * world)
            out_c, grads_c = run(latent, full_grad, None)
            out_d, grads_d = run(latent, full_grad, barrier_between)
            ffm.set_ep_static_forward(None)
            assert torch.equal(out_c, out_a) and torch.equal(out_d, out_a)
            for i, (a, c, d) in enumerate(zip(grads_a, grads_c, grads_d)):
                assert torch.equal(a, c) and torch.equal(a, d), f"static path: gradient {i} differs"
            ffm.set_ep_group(None)
            ws = [(gw.clone().requires_grad_(), wu.clone().requires_grad_(), wd.clone().requires_grad_())
                  for gw, wu, wd, _ in full]
            xs = x.clone().requires_grad_()
            h = xs
            for gw, wu, wd in ws:
                y, _ = ffm.fused_moe(h, gw, wu, wd, top_k=k, expert_bias=bias)
                h = h + y
            (h.float() * go.float()).sum().backward()
            assert rel(out_a, h) <= 1e-6
            assert rel(grads_a[0], xs.grad) <= TOL, f"stack dH {rel(grads_a[0], xs.grad)}"
            for li, (gw, wu, wd) in enumerate(ws):
                fu, fd = wu.grad.float().clone(), wd.grad.float().clone()
                dist.all_reduce(fu)
                dist.all_reduce(fd)
                assert rel(grads_a[1 + 3 * li + 1], fu[rank * El:(rank + 1) * El] / world) <= TOL, f"layer {li} dW_up"
                assert rel(grads_a[1 + 3 * li + 2], fd[rank * El:(rank + 1) * El] / world) <= TOL, f"layer {li} dW_down"


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
    assert rel(hp.grad, route_only) <= TOL, f"routing-only dH {rel(hp.grad, route_only)}"

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
    assert rel(hq.grad, route_only.float() + xs.grad) <= TOL, f"dH with shared expert {rel(hq.grad, route_only.float() + xs.grad)}"

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
    # latent projection gradients against an fp32 restatement of the reference's formulas (fused_moe.py:988-999):
    # every rank regenerates all ranks' tokens (seeded) and simulates the whole group
    ref_lwu, ref_lwd, ref_wu, ref_wd = latent_reference(rank, world, D, E, k, g, wu, wd, lwd, lwu, dev)
    errs = {"d proj_up": rel(lwup.grad, ref_lwu), "d proj_down": rel(lwdp.grad, ref_lwd),
            "dW_up (latent)": rel(wul.grad, ref_wu[rank * El:(rank + 1) * El]),
            "dW_down (latent)": rel(wdl.grad, ref_wd[rank * El:(rank + 1) * El])}
    assert all(v <= TOL for v in errs.values()), errs
    hl = h.clone().requires_grad_()
    out_lf, _ = ffm.fused_moe(hl, g, wu_l, wd_l, top_k=k, ep_group=group, latent_weights=(lwd, lwu),
                              ep_full_input_grad=True)
    (out_lf.float() * go.float()).sum().backward()
    assert torch.equal(out_lf, out_l.detach()) and torch.isfinite(hl.grad).all()
    assert (hl.grad.float() - route_only.to(dev).float()).abs().max() > 0, "latent path adds the expert input gradient"

    # ---- two layers back to back, skewed load: receive regions are reused across layers -------------------------
    stacked_layers_case(rank, world, group, dev)

    # ---- host-sync-free training step: bit for bit the host-planned path, eager and replayed from a CUDA graph ---
    if fm._EP_TRANSPORT == "p2p":
        def train(tokens, grad_out, full):
            ps = [t.clone().requires_grad_() for t in (tokens, g, wu_l, wd_l, sg, su, sd)]
            out, m = ffm.fused_moe(ps[0], ps[1], ps[2], ps[3], top_k=k, ep_group=group, aux_loss_coeff=0.01,
                                   z_loss_coeff=0.001, shared_expert_weights=tuple(ps[4:]), ep_full_input_grad=full,
                                   return_metrics=True)
            ((out.float() * grad_out.float()).sum() + m["aux_loss"] + m["z_loss"]).backward()
            return [out.detach(), m["tokens_per_expert"]] + [p.grad for p in ps]

        bound = 384 + 64 * world
        for full in (False, True):
            want = train(h, go, full)
            ffm.set_ep_static_forward(bound)
            got = [train(h, go, full) for _ in range(2)]
            ffm.set_ep_static_forward(None)
            ops.check_status()
            for run in got:
                for i, (a_, b_) in enumerate(zip(run, want)):
                    assert torch.equal(a_, b_), f"static training differs from the host-planned path (tensor {i}, full={full})"
        # a declared bound on the rows a rank may receive: generous -> same results; too small -> the call moves
        # nothing, status 106 on every rank, nothing stored out of bounds, and the next call works again
        want = train(h, go, True)
        ffm.set_ep_static_forward(bound, max_recv_rows=(3 * k * bound) // 2)
        got = train(h, go, True)
        ops.check_status()
        for i, (a_, b_) in enumerate(zip(got, want)):
            assert torch.equal(a_, b_), f"bounded static mode differs (tensor {i})"
        # (four times the tokens: every expert then needs several 256-row segments, far beyond 64 rows + one segment each)
        ffm.set_ep_static_forward(4 * bound, max_recv_rows=64)
        with torch.no_grad():
            ffm.fused_moe(torch.cat([h] * 4), g, wu_l, wd_l, top_k=k, ep_group=group)
        torch.cuda.synchronize()
        try:
            ops.check_status()
            raise AssertionError("an overflow of the declared bound must set the status word")
        except RuntimeError as exc:
            assert "106" in str(exc), str(exc)
        ffm.set_ep_static_forward(bound)
        got = train(h, go, True)
        ops.check_status()
        for i, (a_, b_) in enumerate(zip(got, want)):
            assert torch.equal(a_, b_), f"static mode after an overflow differs (tensor {i})"
        # one captured step, replayed on other tokens
        ffm.set_ep_static_forward(bound)
        statics = [t.clone().requires_grad_() for t in (h, g, wu_l, wd_l, sg, su, sd)]
        go_static = go.clone()
        cell = {}

        def captured_step():
            for p in statics:
                p.grad = None
            out, _ = ffm.fused_moe(statics[0], statics[1], statics[2], statics[3], top_k=k, ep_group=group,
                                   shared_expert_weights=tuple(statics[4:]), ep_full_input_grad=True)
            (out.float() * go_static.float()).sum().backward()
            cell["out"] = out.detach()

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                captured_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured_step()
        torch.manual_seed(700 + rank)
        h2 = torch.randn(N, D).bfloat16().to(dev)
        go2 = torch.randn(N, D).bfloat16().to(dev)
        for tok, gr in ((h, go), (h2, go2), (h, go)):
            with torch.no_grad():
                statics[0].copy_(tok)
                go_static.copy_(gr)
            graph.replay()
            torch.cuda.synchronize()
            ffm.set_ep_static_forward(None)
            ps = [t.clone().requires_grad_() for t in (tok, g, wu_l, wd_l, sg, su, sd)]
            out_e, _ = ffm.fused_moe(ps[0], ps[1], ps[2], ps[3], top_k=k, ep_group=group,
                                     shared_expert_weights=tuple(ps[4:]), ep_full_input_grad=True)
            (out_e.float() * gr.float()).sum().backward()
            ffm.set_ep_static_forward(bound)
            assert torch.equal(cell["out"], out_e), "replayed training step: output"
            for a_, b_ in zip(statics, ps):
                assert torch.equal(a_.grad, b_.grad), "replayed training step: gradient"
        ops.check_status()
        ffm.set_ep_static_forward(None)
        del graph

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
