"""Real-gated linear recurrent unit and the Hawk block (Griffin, https://arxiv.org/abs/2402.19427).
Reference: ohara/modules/linear_rnn.py:16-110."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .pscan import pscan


def scan(x: Tensor, h: Tensor) -> Tensor:
    """Linear recurrence over dim 1 for ``(B, L, D)`` tensors: ``x`` holds the coefficients and
    ``h`` the driven inputs (the reference's parameter names, ohara/modules/linear_rnn.py:16-20)."""
    return pscan(x, h)


def _trunc_normal(weight: Tensor, std: float, bound: float | None = None) -> None:
    bound = bound if bound is not None else 3 * std
    nn.init.trunc_normal_(weight, mean=0.0, std=std, a=-bound, b=bound)


class RG_LRU(nn.Module):
    """``h_t = a_t h_{t-1} + sqrt(1 - a_t²) (i_t ⊙ x_t)`` with ``a_t = exp(-c softplus(Λ) r_t)``,
    input gate ``i_t`` and recurrence gate ``r_t`` sigmoid projections of ``x_t``, ``c = 8``.
    The recurrence runs over the time steps, as in the paper (the reference transposes steps and
    width before its scan, ohara/modules/linear_rnn.py:40, which makes its unit memoryless).
    ``scan_over_width = True`` (class or instance attribute) reproduces the reference's function,
    for checkpoints that were trained with it."""

    scan_over_width = False

    def __init__(self, dim: int):
        super().__init__()
        self.dim = dim
        self.input_proj = nn.Linear(dim, dim)
        self.gate_proj = nn.Linear(dim, dim)
        self.forget_lambda = nn.Parameter(torch.linspace(-4.323, -9, dim))
        self.C = 8
        self.reset_parameters()

    def forward(self, x: Tensor, *args, **kwargs) -> Tensor:
        recurrence = self.gate_proj(x).sigmoid()
        alpha = (-self.C * F.softplus(self.forget_lambda) * recurrence).exp()
        driven = (1 - alpha**2 + 1e-6).sqrt() * self.input_proj(x).sigmoid() * x
        if self.scan_over_width:
            return scan(alpha.mT.contiguous(), driven.mT.contiguous()).mT
        return scan(alpha, driven)

    def reset_parameters(self, init_std=None) -> None:
        std = init_std or self.dim**-0.5
        for layer in (self.input_proj, self.gate_proj):
            _trunc_normal(layer.weight, std)


class Hawk(nn.Module):
    """Gated block: ``out(gelu(gate) ⊙ RG_LRU(causal_conv(x)))``."""

    def __init__(self, *, dim: int = 1024, expansion_factor: float = 1.5, kernel_size: int = 4):
        super().__init__()
        self.dim = dim
        self.hidden = int(dim * expansion_factor)
        self.proj = nn.Linear(dim, 2 * self.hidden, bias=False)
        self.conv = nn.Conv1d(self.hidden, self.hidden, kernel_size=kernel_size, bias=True,
                              groups=self.hidden, padding=kernel_size - 1)
        self.linear_rnn = RG_LRU(self.hidden)
        self.output = nn.Linear(self.hidden, dim, bias=False)
        self.reset_parameters()

    def forward(self, x: Tensor) -> Tensor:
        steps = x.shape[1]
        gate, branch = self.proj(x).chunk(2, dim=-1)
        branch = self.conv(branch.mT)[..., :steps].mT
        return self.output(F.gelu(gate) * self.linear_rnn(branch))

    def reset_parameters(self, init_std=None) -> None:
        std = init_std or self.dim**-0.5
        _trunc_normal(self.proj.weight, std)
        _trunc_normal(self.output.weight, self.hidden**-0.5, bound=3 * std)


class Griffin(nn.Module):
    """Placeholder kept for API parity: the reference declares the class without a body
    (ohara/modules/linear_rnn.py:107-110)."""
