"""MoELayer: nn.Module wrapper over fused_moe() with the reference's constructor, parameter names and
return value (reference: src/flashfusemoe/nn.py:47-176).

Parameter names match the reference so that state dicts interchange: gate.weight, w_up, w_down,
shared_expert.{w_gate,w_up,w_down}.weight, proj_down.weight, proj_up.weight.
"""

import math

import torch
import torch.nn as nn

from .fused_moe import fused_moe, glu_ffn, set_ep_group


class _GLUFFN(nn.Module):
    """GLU feed-forward used as the shared expert (reference: nn.py:22-44); runs on the library's dense
    GEMM kernels. "geglu" here is the exact (erf) GELU, as in the reference's shared expert."""

    def __init__(self, d_model, ffn_dim, activation="swiglu"):
        super().__init__()
        intermediate = ffn_dim // 2
        self.w_gate = nn.Linear(d_model, intermediate, bias=False)
        self.w_up = nn.Linear(d_model, intermediate, bias=False)
        self.w_down = nn.Linear(intermediate, d_model, bias=False)
        self.activation = activation

    def forward(self, x):
        if self.activation not in ("swiglu", "geglu", "relu_squared"):
            raise ValueError(f"Unknown activation: {self.activation}")
        act = "geglu_erf" if self.activation == "geglu" else self.activation
        lead = x.shape[:-1]
        y = glu_ffn(x.reshape(-1, x.shape[-1]), self.w_gate.weight, self.w_up.weight, self.w_down.weight, act)
        return y.reshape(*lead, y.shape[-1])


class MoELayer(nn.Module):
    """Fused Mixture-of-Experts layer; returns (output, losses) with losses a dict.

    `shared_ffn_dim` (extension, default None = ffn_dim as in the reference, nn.py:103-104) sets the width of
    the single shared GLU FFN, e.g. num_shared_experts * ffn_dim for models whose shared experts are merged.
    `ep_full_input_grad` (extension, default False = the reference's contract) adds the expert input gradient to
    the expert-parallel backward through a reverse dispatch exchange.
    """

    def __init__(self, d_model, ffn_dim, num_experts, top_k=2, activation="swiglu", gating="softmax",
                 num_shared_experts=0, latent_dim=None, capacity_factor=None, max_tokens_per_expert=None,
                 allow_dropped_tokens=True, aux_loss_coeff=0.0, z_loss_coeff=0.0, recompute_activations=False,
                 shared_ffn_dim=None, ep_full_input_grad=False):
        super().__init__()
        self.d_model = d_model
        self.ffn_dim = ffn_dim
        self.num_experts = num_experts
        self.top_k = top_k
        self.activation = activation
        self.gating = gating
        self.half_ffn = ffn_dim // 2
        self.max_tokens_per_expert = max_tokens_per_expert
        self.allow_dropped_tokens = allow_dropped_tokens
        self.aux_loss_coeff = aux_loss_coeff
        self.z_loss_coeff = z_loss_coeff
        self.capacity_factor = capacity_factor
        self.recompute_activations = recompute_activations
        self.ep_full_input_grad = ep_full_input_grad
        self._ep_group = None
        self._ep_size = 1

        self.gate = nn.Linear(d_model, num_experts, bias=False)
        nn.init.kaiming_uniform_(self.gate.weight, a=math.sqrt(5))
        self.gate.weight.data *= 0.01

        self.w_up = nn.Parameter(torch.empty(num_experts, ffn_dim, d_model))
        self.w_down = nn.Parameter(torch.empty(num_experts, d_model, self.half_ffn))
        for e in range(num_experts):
            nn.init.kaiming_uniform_(self.w_up.data[e], a=math.sqrt(5))
            nn.init.kaiming_uniform_(self.w_down.data[e], a=math.sqrt(5))

        if num_shared_experts > 0:
            self.shared_expert = _GLUFFN(d_model, shared_ffn_dim or ffn_dim, activation)
        else:
            self.shared_expert = None

        self.latent_dim = latent_dim
        if latent_dim is not None:
            self.proj_down = nn.Linear(d_model, latent_dim, bias=False)
            self.proj_up = nn.Linear(latent_dim, d_model, bias=False)

    def forward(self, x):
        """x [*, D] -> ([*, D], dict)."""
        leading = x.shape[:-1]
        D = x.shape[-1]
        x_flat = x.reshape(-1, D)

        shared_weights = None
        shared_local = None
        if self.shared_expert is not None:
            if self._ep_group is not None:
                # EP: the shared expert runs inside fused_moe on a side stream (reference: nn.py:126-132)
                shared_weights = (self.shared_expert.w_gate.weight, self.shared_expert.w_up.weight,
                                  self.shared_expert.w_down.weight)
            else:
                # single GPU: fused_moe runs it on a side stream beside the routing kernels, adds its output inside the
                # combine kernel and starts its backward GEMMs with the backward pass
                se = self.shared_expert
                if se.activation not in ("swiglu", "geglu", "relu_squared"):
                    raise ValueError(f"Unknown activation: {se.activation}")
                shared_local = (se.w_gate.weight, se.w_up.weight, se.w_down.weight,
                                "geglu_erf" if se.activation == "geglu" else se.activation)

        latent_weights = None
        if self.latent_dim is not None:
            latent_weights = (self.proj_down.weight, self.proj_up.weight)

        out, losses = fused_moe(
            x_flat, self.gate.weight, self.w_up, self.w_down, self.top_k,
            activation=self.activation, gating=self.gating, capacity_factor=self.capacity_factor,
            aux_loss_coeff=self.aux_loss_coeff, z_loss_coeff=self.z_loss_coeff,
            recompute_activations=self.recompute_activations,
            max_tokens_per_expert=self.max_tokens_per_expert, allow_dropped_tokens=self.allow_dropped_tokens,
            shared_expert_weights=shared_weights, latent_weights=latent_weights,
            ep_full_input_grad=self.ep_full_input_grad, _shared=shared_local)
        return out.reshape(*leading, D), losses

    def shard_experts(self, ep_group, ep_backend="nccl"):
        """Keep only this rank's experts. Call before creating the optimizer (reference: nn.py:163-171)."""
        from .distributed import shard_expert_weights
        self.w_up, self.w_down = shard_expert_weights(self.w_up, self.w_down, ep_group)
        self._ep_group = ep_group
        self._ep_size = torch.distributed.get_world_size(ep_group)
        set_ep_group(ep_group, backend=ep_backend)

    @property
    def expert_params(self):
        """Parameters sharded across EP ranks (excluded from dense gradient sync)."""
        return [self.w_up, self.w_down]
