"""Loop mixture-of-experts: a ModuleList of feed-forward experts, one contiguous slice per expert.

State-dict layout ``experts.E.{up,down,gate}.weight``, ``gate.weight``, ``router_bias`` matches the
reference (ohara/modules/moe.py:10-210). Routing and balancing live in :mod:`.routing`.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200.modules.mlp import MLP_MAP, Linear
from ohara_b200.modules.routing import (  # noqa: F401  (public re-exports)
    QuantileBalancedRouter,
    apply_qb_update,
    expert_load,
    is_recomputing,
    maximal_violation,
    route_tokens,
    router_logits,
)


class MoE(QuantileBalancedRouter):
    def __init__(self, dim: int, hidden_dim: int | None = None, num_experts: int = 4,
                 num_experts_per_tok: int = 2, mlp: str = "swiglu", gate_fn: str = "softmax",
                 quantile_balancing: bool = True):
        super().__init__()
        if not 1 <= num_experts_per_tok <= num_experts:
            raise AssertionError("num_experts_per_tok must be in [1, num_experts]")
        if quantile_balancing and num_experts_per_tok >= num_experts:
            raise AssertionError(
                "quantile balancing reads the (k+1)-th logit as a threshold, so it needs "
                f"num_experts_per_tok < num_experts (got {num_experts_per_tok} == {num_experts})"
            )
        if gate_fn not in ("softmax", "sigmoid"):
            raise AssertionError("gate_fn must be 'softmax' or 'sigmoid'")
        self.dim = dim
        self.hidden_dim = hidden_dim
        self.num_experts = num_experts
        self.num_experts_per_tok = num_experts_per_tok
        self.gate_fn = gate_fn
        self.quantile_balancing = quantile_balancing
        block = MLP_MAP[mlp]
        self.experts = nn.ModuleList([block(dim, hidden_dim) for _ in range(num_experts)])
        self.gate = Linear(dim, num_experts, bias=False)
        self._register_balancing_buffers()

    def forward(self, x: Tensor) -> Tensor:
        batch, seq, dim = x.shape
        flat = x.reshape(batch * seq, dim)
        logits = router_logits(flat, self.gate.weight)
        indices, weights, alpha = route_tokens(
            logits, self.router_bias, self.num_experts_per_tok, self.gate_fn,
            self.quantile_balancing,
        )
        out = self._dispatch(flat, indices, weights.to(x.dtype))
        if self.training and not is_recomputing():
            if self.quantile_balancing:
                self._accumulate_qb(logits.detach(), alpha.detach())
            self._record_load(indices.detach())
        return out.view(batch, seq, dim)

    @torch.no_grad()
    def reset_parameters(self, init_std: float | None = None) -> None:
        """Truncated-normal router (std ``dim ** -0.5`` unless given), zero selection bias, and
        every expert's own ``reset_parameters`` (reference: ohara/modules/moe.py:164-177)."""
        std = init_std or self.dim ** -0.5
        nn.init.trunc_normal_(self.gate.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
        self.router_bias.zero_()
        for expert in self.experts:
            if hasattr(expert, "reset_parameters"):
                expert.reset_parameters(init_std=init_std)

    def _dispatch(self, flat: Tensor, indices: Tensor, weights: Tensor) -> Tensor:
        k = self.num_experts_per_tok
        pair_expert = indices.reshape(-1)
        order = torch.argsort(pair_expert, stable=True)
        token_of_pair = order.div(k, rounding_mode="floor")
        pair_weight = weights.reshape(-1)[order].unsqueeze(-1)
        counts = torch.bincount(pair_expert, minlength=self.num_experts).tolist()
        out = torch.zeros_like(flat)
        begin = 0
        for expert, count in zip(self.experts, counts):
            if count == 0:
                continue
            rows = token_of_pair[begin : begin + count]
            y = expert(flat[rows]) * pair_weight[begin : begin + count].to(flat.dtype)
            out.index_add_(0, rows, y.to(out.dtype))
            begin += count
        return out
