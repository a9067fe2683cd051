"""Pins oracle/moe_oracle.py against the unmodified reference and writes the golden vectors.

Runs only where the reference checkout is available (its directory is the first argument, or the environment
variable FFM_REFERENCE_DIR); it is never imported by tests, bench.py or the package. The reference's Triton kernels run
through Triton's CPU interpreter; its autotuner is told to run each candidate once.

    python oracle/pin_against_reference.py [reference_dir]

Outputs: tests/golden/routing_rule.pt, tests/golden/layer_small_fp32.pt, tests/golden/layer_small_bf16.pt,
tests/golden/layer_config1_fp32.pt (sub-sampled weight gradients), tests/golden/layer_variants_fp32.pt,
tests/golden/module_state_dict_layout.json, tests/golden/module_checkpoint_bf16.pt, and a printed table of oracle-vs-reference
errors that must all be within the bounds asserted below.
"""

import importlib.util
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FFM_REFERENCE_DIR")
if not REF or not os.path.isdir(os.path.join(REF, "src")):
    raise SystemExit("usage: python oracle/pin_against_reference.py <reference checkout>  (or set FFM_REFERENCE_DIR)")
sys.path.insert(0, os.path.join(REF, "src"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
from triton.runtime import autotuner as _at  # noqa: E402

_at.Autotuner.do_bench = property(lambda self: (lambda kernel_call, quantiles=None: (kernel_call(), [1.0, 1.0, 1.0])[1]))

import flashfusemoe  # noqa: E402,F401
from flashfusemoe.kernels.fused_topk import fused_topk_routing  # noqa: E402

ref_mod = sys.modules["flashfusemoe.fused_moe"]
from oracle import moe_oracle as orc  # noqa: E402

GOLD = os.path.join(ROOT, "tests", "golden")
os.makedirs(GOLD, exist_ok=True)


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def pin_routing_rule():
    """Triton top-k kernels (interpreted) vs oracle.route: indices bit-exact, weights to fp32 round-off."""
    torch.manual_seed(7)
    cases = []
    # explicit ties
    lg = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0, 0.0, 2.0, 2.0], [0, 0, 0, 0, 0, 0, 0, 0.0],
                       [-1, -1, 5, 5, -1, 5, 5, -1.0]])
    cases.append(("ties_e8_k3", lg, 3))
    cases.append(("rand_e8_k2_bf16", (torch.randn(64, 8) * 0.5).bfloat16(), 2))
    cases.append(("rand_e64_k6_bf16", (torch.randn(48, 64) * 0.3).bfloat16(), 6))
    cases.append(("coarse_e256_k8_bf16", (torch.randn(32, 256) * 0.05).bfloat16(), 8))  # many bf16 ties
    cases.append(("rand_e24_k3_fp32", torch.randn(40, 24), 3))
    gold = {}
    for name, logits, k in cases:
        for gating in ("softmax", "sigmoid"):
            w_ref, i_ref = fused_topk_routing(logits, gating, k)
            w_o, i_o = orc.route(logits, gating, k)
            assert torch.equal(i_ref, i_o), f"{name}/{gating}: indices differ from the reference kernel"
            assert torch.allclose(w_ref, w_o, atol=1e-6, rtol=1e-5), f"{name}/{gating}: weights differ"
            gold[f"{name}/{gating}"] = dict(logits=logits, k=k, gating=gating, idx=i_ref.to(torch.int32), w=w_ref)
        print(f"routing rule {name}: indices bit-exact for softmax and sigmoid")
    torch.save(gold, os.path.join(GOLD, "routing_rule.pt"))


def make_inputs(seed, N, D, E, F, dtype):
    torch.manual_seed(seed)
    h = torch.randn(N, D)
    g = torch.randn(E, D) * 0.02
    wu = torch.randn(E, F, D) * 0.02
    wd = torch.randn(E, D, F // 2) * 0.02
    go = torch.randn(N, D)
    return [t.to(dtype) for t in (h, g, wu, wd, go)]


def run_reference(h, g, wu, wd, go, k, activation, gating, aux, z, **extra):
    h, g, wu, wd = [t.clone().requires_grad_() for t in (h, g, wu, wd)]
    kw = dict(allow_dropped_tokens=True, max_tokens_per_expert=h.shape[0] * k)
    if "capacity_factor" in extra:
        kw = dict(allow_dropped_tokens=True)
    out, losses = ref_mod.fused_moe(h, g, wu, wd, top_k=k, activation=activation, gating=gating,
                                    aux_loss_coeff=aux, z_loss_coeff=z, return_metrics=True, **kw, **extra)
    loss = (out.float() * go.float()).sum()
    for name in ("aux_loss", "z_loss"):
        if name in losses:
            loss = loss + losses[name]
    loss.backward()
    return dict(out=out.detach(), losses={n: v.detach() for n, v in losses.items()},
                dH=h.grad, dGate=g.grad, dW_up=wu.grad, dW_down=wd.grad)


def run_oracle(h, g, wu, wd, go, k, activation, gating, aux, z, dtype, **extra):
    fw = orc.fused_moe_forward(h, g, wu, wd, k, activation, gating, aux, z, dtype=dtype, **extra)
    bw = orc.fused_moe_backward(fw, go)
    return fw, bw


def pin_layer(tag, seed, N, D, E, F, k, dtype, tol, combos, save_full=True):
    h, g, wu, wd, go = make_inputs(seed, N, D, E, F, dtype)
    gold = dict(seed=seed, shape=(N, D, E, F, k), dtype=str(dtype), cases={})
    if save_full:
        gold["inputs"] = dict(h=h, g=g, wu=wu, wd=wd, go=go)
    for activation, gating, aux, z in combos:
        ref = run_reference(h, g, wu, wd, go, k, activation, gating, aux, z)
        fw, bw = run_oracle(h, g, wu, wd, go, k, activation, gating, aux, z, dtype)
        tpe = torch.bincount(fw["topk_idx"].reshape(-1), minlength=E)
        assert torch.equal(ref["losses"]["tokens_per_expert"].long(), tpe), f"{tag}: expert counts differ"
        errs = dict(out=rel(fw["out"], ref["out"]), dH=rel(bw["dH"], ref["dH"]), dGate=rel(bw["dGate"], ref["dGate"]),
                    dW_up=rel(bw["dW_up"], ref["dW_up"]), dW_down=rel(bw["dW_down"], ref["dW_down"]))
        for name in ("aux_loss", "z_loss"):
            if name in ref["losses"]:
                errs[name] = abs(float(fw["losses"][name]) - float(ref["losses"][name])) / (abs(float(ref["losses"][name])) + 1e-12)
        print(f"{tag} {activation:13s} {gating:8s} aux={aux} z={z}: " + " ".join(f"{n}={v:.1e}" for n, v in errs.items()))
        for n, v in errs.items():
            assert v <= tol, f"{tag}/{activation}/{gating}: {n} off by {v}"
        case = dict(out=ref["out"], dH=ref["dH"], dGate=ref["dGate"], topk_idx=fw["topk_idx"].to(torch.int32),
                    tokens_per_expert=tpe.to(torch.int32),
                    losses={n: float(v) for n, v in ref["losses"].items() if n in ("aux_loss", "z_loss")})
        if save_full:
            case["dW_up"], case["dW_down"] = ref["dW_up"], ref["dW_down"]
        else:  # keep the fixture small: every 8th row / column of the weight gradients
            case["dW_up_s8"], case["dW_down_s8"] = ref["dW_up"][:, ::8, ::8].contiguous(), ref["dW_down"][:, ::8, ::8].contiguous()
        gold["cases"][f"{activation}/{gating}/{aux}/{z}"] = case
    torch.save(gold, os.path.join(GOLD, f"{tag}.pt"))


def pin_variants():
    """Routing enhancements and capacity dropping (reference slow path, fp32): indices, outputs and gradients."""
    N, D, E, F, k = 96, 64, 16, 128, 4
    h, g, wu, wd, go = make_inputs(21, N, D, E, F, torch.float32)
    g = g * 20.0  # spread the logits so that the softmax probabilities differ clearly
    torch.manual_seed(5)
    bias = torch.randn(E) * 0.3
    variants = {
        "capacity_1.0": dict(capacity_factor=1.0),
        "capacity_0.5_sigmoid": dict(capacity_factor=0.5, gating="sigmoid"),
        "expert_bias": dict(expert_bias=bias),
        "pre_softmax": dict(pre_softmax=True),
        "pre_softmax_bias_scale": dict(pre_softmax=True, expert_bias=bias * 0.05, scoring_factor=2.5),
        "groups_4_2": dict(n_group=4, topk_group=2),
        "groups_4_2_sigmoid_bias": dict(n_group=4, topk_group=2, gating="sigmoid", expert_bias=bias * 0.2),
        "groups_8_4_pre_softmax": dict(n_group=8, topk_group=4, pre_softmax=True),
    }
    gold = dict(seed=21, shape=(N, D, E, F, k), gate_scale=20.0, bias=bias, cases={})
    for name, extra in variants.items():
        extra = dict(extra)
        gating = extra.pop("gating", "softmax")
        ref = run_reference(h, g, wu, wd, go, k, "swiglu", gating, 0.0, 0.0, **extra)
        fw, bw = run_oracle(h, g, wu, wd, go, k, "swiglu", gating, 0.0, 0.0, torch.float32, **extra)
        errs = dict(out=rel(fw["out"], ref["out"]), dH=rel(bw["dH"], ref["dH"]), dGate=rel(bw["dGate"], ref["dGate"]),
                    dW_up=rel(bw["dW_up"], ref["dW_up"]), dW_down=rel(bw["dW_down"], ref["dW_down"]))
        print(f"variant {name:26s}: " + " ".join(f"{n}={v:.1e}" for n, v in errs.items()))
        for n, v in errs.items():
            assert v <= 2e-5, f"variant {name}: {n} off by {v}"
        case = dict(gating=gating, extra={a: b for a, b in extra.items() if a != "expert_bias"},
                    has_bias="expert_bias" in extra, bias_scale=float((extra["expert_bias"] / bias).mean()) if "expert_bias" in extra else 0.0,
                    out=ref["out"], dH=ref["dH"], dGate=ref["dGate"], topk_idx=fw["topk_idx"].to(torch.int32),
                    topk_w=fw["topk_w"])
        if "capacity_factor" in extra:
            case["dropped"] = int(ref["losses"]["dropped_token_count"])
            assert case["dropped"] == int((fw["keep"] == 0).sum()), name
        gold["cases"][name] = case
    torch.save(gold, os.path.join(GOLD, "layer_variants_fp32.pt"))


def pin_module():
    """Reference MoELayer: parameter names and shapes per constructor variant, and one bf16 checkpoint with a shared
    expert run forward + backward through the unmodified module (checkpoint interchange, nn.py:56-176)."""
    import json
    from flashfusemoe import MoELayer as RefLayer
    variants = {
        "base": dict(),
        "shared": dict(num_shared_experts=1),
        "latent": dict(latent_dim=32),
        "shared_latent_sigmoid": dict(num_shared_experts=2, latent_dim=32, gating="sigmoid", activation="geglu"),
    }
    layout = {}
    for name, kw in variants.items():
        layer = RefLayer(64, 128, 8, 2, **kw)
        layout[name] = dict(kwargs=kw, params={n: list(t.shape) for n, t in layer.state_dict().items()})
    with open(os.path.join(GOLD, "module_state_dict_layout.json"), "w") as f:
        json.dump(layout, f, indent=1, sort_keys=True)

    torch.manual_seed(31)
    layer = RefLayer(64, 128, 8, 2, num_shared_experts=1, aux_loss_coeff=0.01, z_loss_coeff=0.001)
    with torch.no_grad():
        for prm in layer.parameters():
            prm.normal_(0.0, 0.05)
    layer = layer.bfloat16()
    x = torch.randn(2, 48, 64).bfloat16().requires_grad_()
    go = torch.randn(2, 48, 64).bfloat16()
    out, losses = layer(x)
    loss = (out.float() * go.float()).sum() + losses["aux_loss"] + losses["z_loss"]
    loss.backward()
    gold = dict(ctor=dict(d_model=64, ffn_dim=128, num_experts=8, top_k=2, num_shared_experts=1, aux_loss_coeff=0.01,
                          z_loss_coeff=0.001),
                state_dict={n: t.detach().clone() for n, t in layer.state_dict().items()},
                x=x.detach().clone(), go=go, out=out.detach().clone(), dx=x.grad.clone(),
                losses={n: float(v.detach()) for n, v in losses.items() if n in ("aux_loss", "z_loss")},
                grads={n: prm.grad.clone() for n, prm in layer.named_parameters()})
    torch.save(gold, os.path.join(GOLD, "module_checkpoint_bf16.pt"))
    print("module layout and checkpoint written:", sorted(layout["shared_latent_sigmoid"]["params"]))


if __name__ == "__main__":
    pin_routing_rule()
    pin_module()
    pin_variants()
    combos = [("swiglu", "softmax", 0.01, 0.001), ("geglu", "softmax", 0.0, 0.0), ("relu_squared", "sigmoid", 0.01, 0.001),
              ("swiglu", "sigmoid", 0.0, 0.0)]
    pin_layer("layer_small_fp32", 11, 96, 64, 8, 128, 2, torch.float32, 2e-5, combos)
    pin_layer("layer_small_bf16", 12, 96, 64, 8, 128, 2, torch.bfloat16, 2e-2, combos)
    # BASELINE configs[0]: seed 0, fp32, N=512 D=256 E=8 ffn_dim=1024 k=2, swiglu, aux 0.01, z-loss on (coeff 1e-3)
    pin_layer("layer_config1_fp32", 0, 512, 256, 8, 1024, 2, torch.float32, 2e-5, [("swiglu", "softmax", 0.01, 0.001)],
              save_full=False)
    print("oracle pinned against the reference; golden vectors written to", GOLD)
