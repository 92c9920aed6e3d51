"""Swap layers of an existing model for experimental ones (reference:
experiments/template/monkey_patcher.py:62-114 and its copies under mHC/ and springnet/).

``replace_modules`` walks a model and replaces every child for which ``select(name, module)`` is
true by ``build(module)``; ``copy_linear_weights`` carries a linear layer's weights into its
replacement so a patched model starts from the original function. ``DMLinear`` is the
direction / magnitude linear layer the reference's template patches in: rows of the weight are
normalised and a learned per-output scale restores the magnitude."""

from __future__ import annotations

from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor


class DMLinear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True) -> None:
        super().__init__(in_features, out_features, bias)
        self.scale = nn.Parameter(torch.ones(1, out_features))

    def forward(self, x: Tensor) -> Tensor:
        direction = F.normalize(self.weight, dim=1)
        out = F.linear(x, direction) * self.scale
        return out if self.bias is None else out + self.bias

    @classmethod
    def from_linear(cls, linear: nn.Linear) -> "DMLinear":
        """Same function as ``linear``: direction from its rows, scale from their norms."""
        new = cls(linear.in_features, linear.out_features, linear.bias is not None)
        with torch.no_grad():
            new.weight.copy_(linear.weight)
            new.scale.copy_(linear.weight.norm(dim=1)[None])
            if linear.bias is not None:
                new.bias.copy_(linear.bias)
        return new


def replace_modules(model: nn.Module, select: Callable[[str, nn.Module], bool],
                    build: Callable[[nn.Module], nn.Module], prefix: str = "") -> list[str]:
    """Returns the dotted names of the replaced modules."""
    replaced = []
    for name, child in list(model.named_children()):
        path = f"{prefix}{name}"
        if select(path, child):
            setattr(model, name, build(child))
            replaced.append(path)
        else:
            replaced += replace_modules(child, select, build, prefix=f"{path}.")
    return replaced


def patch_linears(model: nn.Module, names: set[str] | None = None,
                  build: Callable[[nn.Linear], nn.Module] = DMLinear.from_linear) -> list[str]:
    """Replace ``nn.Linear`` children whose attribute name is in ``names`` (all of them when
    ``names`` is None)."""
    def select(path: str, module: nn.Module) -> bool:
        return isinstance(module, nn.Linear) and not isinstance(module, DMLinear) and (
            names is None or path.rsplit(".", 1)[-1] in names)

    return replace_modules(model, select, build)
