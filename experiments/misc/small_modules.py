"""Small single-idea modules from the reference's experiments folder.

* ``relu_squared`` - ReLU(x)^2 as an explicit autograd function (experiments/relu_next/
  model_relu_next.py:41-63), and ``silulu = silu(x) + relu(x)^2``.
* ``XLinear`` - a linear layer that multiplies by its weight rows normalised to unit length, so
  only the direction of a row matters (experiments/hypersphere/hs.py:9-30).
* ``Pattention`` - "parameter-token attention": the input attends over learned key / value tokens
  with a GELU + L2 normalisation instead of a softmax, so that tokens can be appended (zero
  initialised) without changing the function (experiments/tokenformer/pattention.py:11-96).
* ``GaLoreProjector`` - projects a gradient onto its top singular subspace, refreshed every
  ``update_gap`` steps, and back (experiments/galore/galore.py:14-221).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor


class _ReLUSquared(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor) -> Tensor:
        ctx.save_for_backward(x)
        return torch.relu(x).square()

    @staticmethod
    def backward(ctx, grad: Tensor) -> Tensor:
        (x,) = ctx.saved_tensors
        return 2.0 * torch.relu(x) * grad


def relu_squared(x: Tensor) -> Tensor:
    return _ReLUSquared.apply(x)


def silulu(x: Tensor) -> Tensor:
    return F.silu(x) + torch.relu(x).square()


class XLinear(nn.Linear):
    def forward(self, x: Tensor) -> Tensor:
        # The reference multiplies the product by the row norms of the *normalised* weight, which
        # are one: the layer's function is the product with unit-length rows (plus the bias).
        norm = self.weight.norm(dim=-1, keepdim=True)
        return F.linear(x, self.weight / norm, self.bias)


def gelu_l2_norm(x: Tensor, dim: int = -1) -> Tensor:
    y = F.gelu(x)
    return y / y.norm(dim=dim, keepdim=True).clamp_min(1e-12) * math.sqrt(y.shape[dim])


class Pattention(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, num_tokens: int) -> None:
        super().__init__()
        self.keys = nn.Parameter(torch.empty(num_tokens, in_dim))
        self.values = nn.Parameter(torch.empty(num_tokens, out_dim))
        nn.init.xavier_uniform_(self.keys)
        nn.init.xavier_uniform_(self.values)

    def forward(self, x: Tensor) -> Tensor:
        return gelu_l2_norm(x @ self.keys.t()) @ self.values

    @torch.no_grad()
    def expand_tokens(self, num_tokens: int) -> None:
        """Grow to ``num_tokens`` parameter tokens; new value tokens are zero, so the new tokens
        contribute nothing until they are trained (the normalisation constant does change)."""
        extra = num_tokens - self.keys.shape[0]
        if extra <= 0:
            raise ValueError("num_tokens must exceed the current number of parameter tokens")
        self.keys = nn.Parameter(torch.cat([self.keys, self.keys.new_zeros(extra, self.keys.shape[1])]))
        self.values = nn.Parameter(
            torch.cat([self.values, self.values.new_zeros(extra, self.values.shape[1])]))


class GaLoreProjector:
    def __init__(self, rank: int, update_gap: int = 200, scale: float = 1.0) -> None:
        if rank < 1 or update_gap < 1 or scale <= 0:
            raise ValueError("rank, update_gap and scale must be positive")
        self.rank, self.update_gap, self.scale = rank, update_gap, scale
        self.basis: Tensor | None = None
        self._left = False

    def project(self, grad: Tensor, step: int) -> Tensor:
        """(out, in) -> (out, rank) when out >= in (right singular vectors), else (rank, in)."""
        if self.basis is None or step % self.update_gap == 0:
            u, _, vt = torch.linalg.svd(grad.float(), full_matrices=False)
            self._left = grad.shape[0] < grad.shape[1]
            basis = u[:, : self.rank] if self._left else vt[: self.rank]
            self.basis = basis.to(grad.dtype)
        return self.basis.t() @ grad if self._left else grad @ self.basis.t()

    def project_back(self, low_rank: Tensor) -> Tensor:
        if self.basis is None:
            raise RuntimeError("project() must run before project_back()")
        full = self.basis @ low_rank if self._left else low_rank @ self.basis
        return full * self.scale
