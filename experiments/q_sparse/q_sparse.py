"""Q-Sparse: keep the K largest activations of every row, pass gradients straight through
(reference: experiments/q_sparse/q_sparse.py:6-50)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor


class _TopKStraightThrough(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, k: int) -> Tensor:
        values, indices = torch.topk(x, k, dim=-1)
        return torch.zeros_like(x).scatter_(-1, indices, values)

    @staticmethod
    def backward(ctx, grad: Tensor):
        return grad, None


def q_sparse(x: Tensor, k: int) -> Tensor:
    return _TopKStraightThrough.apply(x, k)


class QSparseLinear(nn.Linear):
    """Linear layer on the top-``pct`` fraction of its (L2-normalised) input features."""

    def __init__(self, pct: float, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.k = max(1, int(pct * self.in_features))

    def forward(self, x: Tensor) -> Tensor:
        x = q_sparse(x, self.k)
        x = x / x.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        return F.linear(x, self.weight, self.bias)


def patch_linears(model: nn.Module, target_layers: list[str], pct: float = 0.7) -> nn.Module:
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear) and name in target_layers:
            layer = QSparseLinear(pct, child.in_features, child.out_features,
                                  bias=child.bias is not None)
            with torch.no_grad():
                layer.weight.copy_(child.weight)
                if child.bias is not None:
                    layer.bias.copy_(child.bias)
            setattr(model, name, layer)
        else:
            patch_linears(child, target_layers, pct)
    return model
