"""Mixture of depths (reference: experiments/mixture_of_depth/mixture_of_depth.py:73-170).

A scalar router scores every token; only the top ``capacity_factor * seq_len`` tokens of a sequence
go through the wrapped block (in their original order, so a causal block stays causal among them),
the others skip it. The block's output is scaled by the softmax of the selected router scores and
added back. Because top-k over the sequence looks at future tokens, an auxiliary router is trained
(binary cross-entropy on stop-gradient inputs) to predict the selection token by token; it is what
autoregressive inference uses.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor


class MixtureOfDepth(nn.Module):
    def __init__(self, block: nn.Module, dim: int, capacity_factor: float = 0.125) -> None:
        super().__init__()
        if not 0.0 < capacity_factor <= 1.0:
            raise ValueError("capacity_factor must be in (0, 1]")
        self.block, self.capacity_factor = block, capacity_factor
        self.router = nn.Linear(dim, 1, bias=False)
        self.aux_router = nn.Sequential(nn.Linear(dim, dim // 2), nn.SiLU(), nn.Linear(dim // 2, 1))

    def forward(self, x: Tensor, *block_args, auxiliary_loss: bool = False, **block_kwargs):
        b, t, d = x.shape
        k = max(1, int(t * self.capacity_factor))
        logits = self.router(x)                                   # (b, t, 1)
        weights, chosen = torch.topk(logits, k, dim=1, sorted=False)
        chosen, order = torch.sort(chosen, dim=1)                 # back to sequence order
        weights = F.softmax(weights, dim=1).gather(1, order)
        index = chosen.expand(-1, -1, d)
        processed = self.block(x.gather(1, index), *block_args, **block_kwargs)
        if isinstance(processed, tuple):
            processed = processed[0]
        out = x.scatter_add(1, index, weights * processed)
        if not auxiliary_loss:
            return out, None
        targets = torch.zeros(b, t, device=x.device, dtype=logits.dtype).scatter_(1, chosen[..., 0], 1.0)
        predicted = self.aux_router(x.detach()).squeeze(-1)
        return out, F.binary_cross_entropy_with_logits(predicted, targets)

    @torch.no_grad()
    def select_for_decoding(self, x: Tensor) -> Tensor:
        """Token-local decision of the auxiliary router: which positions would enter the block."""
        return self.aux_router(x).squeeze(-1) > 0
