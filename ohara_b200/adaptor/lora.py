"""LoRA (https://arxiv.org/abs/2106.09685): ``y = W x + (alpha/r) B A x``.
API as in the reference (ohara/adaptor/lora.py:9-110)."""

from __future__ import annotations

import torch
import torch.nn as nn

from ._base import (
    LowRankAdapter,
    adapter_from_linear,
    mark_only_adapters_trainable,
    merge_adapters,
    replace_linears,
)


class LoRALinear(LowRankAdapter):
    enable_lora = True

    def reset_lora_parameters(self, lora_only: bool = False) -> None:
        self.reset_adapter_parameters()

    def lora_trainable_only(self) -> None:
        self.adapter_trainable_only()

    @torch.no_grad()
    def merge(self) -> None:
        if not self.merged and self.rank > 0:
            self.linear.weight.data += self.delta()
            self.merged = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = self.linear(x)
        if self.rank == 0 or self.merged:
            return out
        return out + (self.lora_dropout(x) @ self.lora_A.T @ self.lora_B.T) * self.scaling


def lora_from_linear(linear: nn.Linear, lora_alpha: int = 1, lora_dropout: float = 0.0, rank: int = 16):
    return adapter_from_linear(LoRALinear, linear, lora_alpha, lora_dropout, rank)


def replace_with_lora(model: nn.Module, target_layer: list[str] | None = None, lora_alpha: int = 1,
                      lora_dropout: float = 0.0, rank: int = 16):
    return replace_linears(LoRALinear, model, target_layer, lora_alpha, lora_dropout, rank)


def mark_lora_as_trainable(model: nn.Module, target_layer: list[str] | None = None):
    return mark_only_adapters_trainable(LoRALinear, model)


def merge_lora(model: nn.Module, target_layer: list[str] | None = None):
    return merge_adapters(LoRALinear, model)
