"""DeGLU: a feed-forward layer gated by a *fixed random* block mask instead of a learned gate
(reference: "experiments/unmasking divine benevolence/deglu.py":42-70).

The hidden activations are projected by a frozen random matrix to ``mask_blocks`` scores; the
hidden units are cut into ``mask_blocks`` equal blocks and only the block(s) whose softmax score
equals the largest score in the whole batch pass. The mask carries no gradient."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor


class DeGLU(nn.Module):
    def __init__(self, dim: int, hidden_dim: int | None = None, mask_blocks: int = 4,
                 bias: bool = False) -> None:
        super().__init__()
        hidden_dim = hidden_dim or 4 * dim
        if hidden_dim % mask_blocks:
            raise ValueError("hidden_dim must divide into mask_blocks")
        self.mask_blocks = mask_blocks
        self.up = nn.Linear(dim, hidden_dim, bias=bias)
        self.down = nn.Linear(hidden_dim, dim, bias=bias)
        self.register_buffer("mask_proj", torch.randn(hidden_dim, mask_blocks))

    @torch.no_grad()
    def get_mask(self, hidden: Tensor) -> Tensor:
        scores = F.softmax(hidden @ self.mask_proj, dim=-1)
        keep = (scores >= scores.max()).to(hidden.dtype)
        return keep.repeat_interleave(hidden.shape[-1] // self.mask_blocks, dim=-1)

    def forward(self, x: Tensor) -> Tensor:
        hidden = F.silu(self.up(x))
        return self.down(hidden * self.get_mask(hidden))
