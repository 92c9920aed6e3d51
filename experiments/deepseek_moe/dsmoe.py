"""DeepSeek-style mixture of experts (reference: experiments/deepseek_moe/dsmoe.py:64-238).

Always-on shared experts plus top-k routed experts. Selection uses ``scores + bias``; the mixing
weights come from the unbiased scores (sigmoid, normalised over the selected experts). Load is
balanced either without an auxiliary loss - after every training forward the bias of an
under-loaded expert goes up by ``expert_update_rate`` and that of an over-loaded one goes down
(sign update) - or with the classic load x importance auxiliary loss.

One deliberate difference: the reference weights the picked experts with the ``k`` largest
unbiased scores in order (dsmoe.py:181), which are the picked experts' own scores only while the
biases do not change the pick; here an expert is always weighted with its own score.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200.modules.mlp import MLP_MAP
from ohara_b200.modules.routing import maximal_violation


class DSMoE(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int | None = None, num_experts: int = 4,
                 experts_per_token: int = 2, num_shared_experts: int = 1,
                 expert_update_rate: float = 1e-3, aux_free_loadbalancing: bool = True,
                 use_aux_loss: bool = False, mlp: str = "swiglu") -> None:
        super().__init__()
        if aux_free_loadbalancing == use_aux_loss:
            raise ValueError("choose exactly one of aux_free_loadbalancing and use_aux_loss")
        block = MLP_MAP[mlp.lower()]
        self.num_experts, self.experts_per_token = num_experts, experts_per_token
        self.expert_update_rate = expert_update_rate
        self.aux_free_loadbalancing, self.use_aux_loss = aux_free_loadbalancing, use_aux_loss
        self.experts = nn.ModuleList(block(hidden_size, intermediate_size) for _ in range(num_experts))
        self.shared_experts = nn.ModuleList(
            block(hidden_size, intermediate_size) for _ in range(num_shared_experts))
        self.gate = nn.Linear(hidden_size, num_experts, bias=False)
        # (the name is the reference's, so that its state dicts load here: dsmoe.py:122)
        self.register_buffer("e_expert_biases", torch.zeros(num_experts))

    @property
    def expert_biases(self) -> Tensor:
        return self.e_expert_biases

    def forward(self, x: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        """Returns ``(output, auxiliary loss, maximal load violation)``."""
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        scores = self.gate(flat)
        indices = torch.topk(scores + self.expert_biases, self.experts_per_token, dim=-1).indices
        weights = scores.gather(-1, indices).sigmoid()
        weights = weights / weights.sum(dim=-1, keepdim=True)
        out = torch.zeros_like(flat)
        for e, expert in enumerate(self.experts):
            token, slot = (indices == e).nonzero(as_tuple=True)
            if token.numel():
                out.index_add_(0, token, expert(flat[token]) * weights[token, slot, None])
        for expert in self.shared_experts:
            out = out + expert(flat)
        counts = torch.bincount(indices.reshape(-1), minlength=self.num_experts)
        aux = scores.detach().new_zeros(())
        if self.use_aux_loss:
            probs = scores.softmax(-1)
            load = counts.to(probs.dtype) / indices.numel()
            aux = self.num_experts * (load * probs.mean(0)).sum()
        if self.training and self.aux_free_loadbalancing:
            frequency = counts.float() / indices.numel()
            self.e_expert_biases += self.expert_update_rate * torch.sign(frequency.mean() - frequency)
        return out.view(shape), aux, maximal_violation(counts)
