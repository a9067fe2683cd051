"""GPU, >= 2 devices: expert parallelism over NCCL (tests/ep_worker.py under torch.distributed.run)."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("transport", ["p2p", "p2p_contiguous", "nccl"])
def test_expert_parallel_two_ranks(transport):
    # p2p: peer stores straight into the receivers' grouped layout; p2p_contiguous: peer stores of one contiguous
    # range per peer with a permute on either side; nccl: torch.distributed all_to_all_single
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", FFM_EP_TRANSPORT=transport.split("_")[0],
               FFM_EP_DIRECT="0" if transport == "p2p_contiguous" else "1", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29511", os.path.join(ROOT, "tests", "ep_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert p.stdout.count("EP_OK") == 2
