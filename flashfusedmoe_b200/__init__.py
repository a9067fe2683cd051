"""B200-native fused Mixture-of-Experts layer (sm_100a kernels behind a C ABI) with the public surface of
FlashFusedMoE (reference: src/flashfusemoe/__init__.py:1-17)."""

from .fused_moe import (fused_moe, set_ep_group, set_aux_loss_grad, set_ep_static_forward,
                        set_expert_gemm_precision)
from .nn import MoELayer
from .expert_parallel import (ExpertParallelDispatcher, MockExpertParallelDispatcher, DispatchHandle,
                              create_dispatcher)
from .distributed import shard_expert_weights, OverlappedGradSync, get_dense_params

__all__ = [
    "fused_moe", "set_ep_group", "MoELayer", "ExpertParallelDispatcher", "MockExpertParallelDispatcher",
    "DispatchHandle", "create_dispatcher", "shard_expert_weights", "OverlappedGradSync", "get_dense_params",
    "set_aux_loss_grad", "set_ep_static_forward", "set_expert_gemm_precision",
]
