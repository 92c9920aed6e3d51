"""DoRA (https://arxiv.org/abs/2402.09353): the adapted weight ``W + (alpha/r) B A`` is
renormalised per output row and rescaled by a learned magnitude vector initialised to the row
norms of ``W``. API as in the reference (ohara/adaptor/dora.py:10-137)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ._base import (
    LowRankAdapter,
    adapter_from_linear,
    mark_only_adapters_trainable,
    merge_adapters,
    replace_linears,
)


class DoRALinear(LowRankAdapter):
    enable_dora = True

    def _register_extra_parameters(self, out_features: int) -> None:
        self.magnitude = nn.Parameter(torch.ones((out_features, 1)))

    def _reset_extra_parameters(self) -> None:
        self.reset_magnitude()

    def _adapter_parameters(self) -> list[nn.Parameter]:
        return [self.lora_A, self.lora_B, self.magnitude]

    @torch.no_grad()
    def reset_magnitude(self) -> None:
        self.magnitude.copy_(torch.norm(self.linear.weight, p=2, dim=1, keepdim=True))

    def reset_dora_parameters(self) -> None:
        self.reset_adapter_parameters()

    def dora_trainable_only(self) -> None:
        self.adapter_trainable_only()

    def _row_scale(self, weight: torch.Tensor) -> torch.Tensor:
        return self.magnitude / torch.norm(weight, p=2, dim=1, keepdim=True).clamp(min=1e-6)

    @torch.no_grad()
    def merge(self) -> None:
        if not self.merged and self.rank > 0:
            weight = self.linear.weight + self.delta()
            self.linear.weight.copy_(weight * self._row_scale(weight))  # in place: bumps the version
            self.merged = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.rank == 0 or self.merged:
            return self.linear(x)
        delta = self.delta()
        scale = self._row_scale(self.linear.weight + delta)
        out = (F.linear(x, self.linear.weight) + F.linear(self.lora_dropout(x), delta)) * scale.T
        if self.linear.bias is not None:
            out = out + self.linear.bias
        return out


def dora_from_linear(linear: nn.Linear, lora_alpha: int = 1, lora_dropout: float = 0.0, rank: int = 16):
    return adapter_from_linear(DoRALinear, linear, lora_alpha, lora_dropout, rank)


def replace_with_dora(model: nn.Module, target_layer: list[str] | None = None, lora_alpha: int = 1,
                      lora_dropout: float = 0.0, rank: int = 16):
    return replace_linears(DoRALinear, model, target_layer, lora_alpha, lora_dropout, rank)


def mark_dora_as_trainable(model: nn.Module, target_layer: list[str] | None = None):
    return mark_only_adapters_trainable(DoRALinear, model)


def merge_dora(model: nn.Module, target_layer: list[str] | None = None):
    return merge_adapters(DoRALinear, model)
