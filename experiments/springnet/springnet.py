"""SpringMLP: one feed-forward layer applied ``spring_steps`` times with a learned, shrinking step
(reference: experiments/springnet/model.py:44-70).

Every iteration predicts a per-token decay in (0, 1) from the current state; the running product
of squared decays ``gamma`` scales that iteration's update ``x += gamma * norm(mlp(x))``, so later
iterations move the state less and less, like a damped spring. The mean ``gamma`` over the
iterations is returned as an auxiliary term: adding it to the loss rewards settling early."""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200.modules.mlp import MLP


class SpringMLP(nn.Module):
    includes_residual = True  # the output is the input moved, not an update to add to it

    def __init__(self, d_model: int, hidden_dim: int, spring_steps: int = 10,
                 dropout: float = 0.0, bias: bool = False) -> None:
        super().__init__()
        self.spring_steps = spring_steps
        self.mlp = MLP(d_model, hidden_dim, dropout=dropout, bias=bias)
        self.norm = nn.LayerNorm(d_model)
        self.decay = nn.Sequential(nn.Linear(d_model, d_model // 2), nn.SiLU(),
                                   nn.Linear(d_model // 2, 1), nn.Sigmoid())

    def forward(self, x: Tensor) -> tuple[Tensor, Tensor]:
        """Returns the settled state and the mean step size ``(batch, steps, 1)``."""
        gamma = torch.ones_like(x[..., :1])
        total = torch.zeros_like(gamma)
        for _ in range(self.spring_steps):
            gamma = gamma * self.decay(x).square()
            total = total + gamma
            x = x + self.norm(self.mlp(x)) * gamma
        return x, total / self.spring_steps

    def step_sizes(self, x: Tensor) -> Tensor:
        """``gamma`` of every iteration, ``(spring_steps, batch, steps, 1)`` (for inspection)."""
        sizes = []
        gamma = torch.ones_like(x[..., :1])
        with torch.no_grad():
            for _ in range(self.spring_steps):
                gamma = gamma * self.decay(x).square()
                sizes.append(gamma)
                x = x + self.norm(self.mlp(x)) * gamma
        return torch.stack(sizes)
