"""XPos rotation + per-head exponential decay mask used by RetNet (https://arxiv.org/abs/2212.10554).

Reference behaviour: ohara/embeddings_pos/xpos.py:7-37.
"""

from __future__ import annotations

import torch
import torch.nn as nn


class XPos(nn.Module):
    def __init__(self, dim: int, num_heads: int) -> None:
        super().__init__()
        angle = 1.0 / (10000 ** torch.linspace(0, 1, dim // num_heads // 2))
        self.register_buffer("angle", angle.repeat_interleave(2))
        self.register_buffer(
            "decay", torch.log(1 - 2 ** (-5 - torch.arange(num_heads, dtype=torch.float)))
        )

    def forward(self, slen: int, recurrent: bool = False):
        """``((cos, sin), decay)``: a ``(heads, T, T)`` normalised decay mask, or the scalar
        per-head decay for the recurrent form."""
        if recurrent:
            phase = self.angle * (slen - 1)
            return (torch.cos(phase), torch.sin(phase)), self.decay.exp()
        index = torch.arange(slen).to(self.decay)
        phase = index[:, None] * self.angle[None, :]
        lower = torch.tril(torch.ones(slen, slen, device=index.device)).bool()
        gap = torch.masked_fill(index[:, None] - index[None, :], ~lower, float("inf"))
        mask = torch.nan_to_num(torch.exp(gap * self.decay[:, None, None]))
        mask = mask / mask.sum(dim=-1, keepdim=True).sqrt()
        return (torch.cos(phase), torch.sin(phase)), mask
