"""bench.py's reference arm and argument handling, on CPU (the GPU arm needs a B200)."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s_fwd_bwd" and d["unit"] == "tokens/s"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype",
                "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["value"] > 0 and d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"] and "model" not in d["config"]


def test_reference_arm_is_silent_on_other_ranks():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps",
                        "1", "--warmup", "1"], capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert p.returncode == 0, p.stderr[-2000:]
    assert not [ln for ln in p.stdout.splitlines() if ln.startswith("{")]


def test_routing_only_input_gradient_restatement_against_the_oracle():
    """bench.py's fp32 restatement of the expert-parallel input gradient (routing-weight path + shared expert, the
    experts' own input held constant: reference fused_moe.py:1001-1005), which `ep_parity` compares the sharded
    layer with, agrees with the oracle's backward on a small case (the oracle rounds to bf16 where the reference
    does, the restatement does not: bf16 bound)."""
    import importlib.util
    import torch
    from oracle import moe_oracle as orc
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    torch.manual_seed(0)
    N, D, E, F, k = 96, 64, 8, 128, 2
    bf = torch.bfloat16
    h = torch.randn(N, D).to(bf)
    g = (torch.randn(E, D) * 0.1).to(bf)
    wu = (torch.randn(E, F, D) * 0.1).to(bf)
    wd = (torch.randn(E, D, F // 2) * 0.1).to(bf)
    shared = [(torch.randn(F // 2, D) * 0.1).to(bf), (torch.randn(F // 2, D) * 0.1).to(bf),
              (torch.randn(D, F // 2) * 0.1).to(bf)]
    go = torch.randn(N, D).to(bf)
    fw = orc.fused_moe_forward(h, g, wu, wd, k, dtype=bf)
    bw = orc.fused_moe_backward(fw, go)
    route_only = orc.mm(bw["gl"], g, bf).float()
    xs = h.float().requires_grad_()
    ws = [t.float() for t in shared]
    ((torch.nn.functional.silu(xs @ ws[0].T) * (xs @ ws[1].T)) @ ws[2].T * go.float()).sum().backward()
    want = route_only + xs.grad
    got = bench.routing_only_input_grad(h, go, g, wu, wd, shared, fw["topk_idx"])
    err = ((got - want).abs().max() / want.abs().max()).item()
    assert err <= 2e-2, err
