"""Checkpoint interchange with the reference's MoELayer (reference: src/flashfusemoe/nn.py:56-176).

The fixtures were written by oracle/pin_against_reference.py from the unmodified reference module:
  module_state_dict_layout.json  parameter names and shapes for four constructor variants
  module_checkpoint_bf16.pt      a bf16 state dict with a shared expert, one input, and the reference's own output,
                                 losses, input gradient and parameter gradients (run on CPU)
"""

import json
import os

import pytest
import torch

import flashfusedmoe_b200 as ffm

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 2e-2  # max|a - b| / max|b| for bf16 outputs and gradients


def rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def test_state_dict_names_and_shapes_match_reference():
    layout = json.load(open(os.path.join(GOLD, "module_state_dict_layout.json")))
    assert len(layout) == 4
    for name, entry in layout.items():
        layer = ffm.MoELayer(64, 128, 8, 2, **entry["kwargs"])
        ours = {n: list(t.shape) for n, t in layer.state_dict().items()}
        assert ours == entry["params"], name


def test_reference_checkpoint_loads_strict_on_cpu():
    gold = torch.load(os.path.join(GOLD, "module_checkpoint_bf16.pt"))
    layer = ffm.MoELayer(**gold["ctor"]).bfloat16()
    missing, unexpected = layer.load_state_dict(gold["state_dict"], strict=True)
    assert not missing and not unexpected
    for n, t in layer.state_dict().items():
        assert torch.equal(t, gold["state_dict"][n]), n


@pytest.mark.gpu
def test_reference_checkpoint_reproduces_reference_outputs():
    from flashfusedmoe_b200 import ops
    gold = torch.load(os.path.join(GOLD, "module_checkpoint_bf16.pt"))
    layer = ffm.MoELayer(**gold["ctor"]).bfloat16()
    layer.load_state_dict(gold["state_dict"], strict=True)
    layer = layer.cuda()
    x = gold["x"].cuda().requires_grad_()
    out, losses = layer(x)
    assert out.shape == gold["out"].shape and out.dtype == torch.bfloat16
    loss = (out.float() * gold["go"].cuda().float()).sum() + losses["aux_loss"] + losses["z_loss"]
    loss.backward()
    ops.check_status()
    assert rel(out, gold["out"]) <= TOL
    assert rel(x.grad, gold["dx"]) <= TOL
    for n in ("aux_loss", "z_loss"):
        assert abs(float(losses[n]) - gold["losses"][n]) <= 2e-2 * abs(gold["losses"][n]) + 1e-7, n
    for n, prm in layer.named_parameters():
        assert prm.grad is not None, n
        assert rel(prm.grad, gold["grads"][n]) <= TOL, n
