"""Shared machinery of the low-rank adapters: wrapping an ``nn.Linear``, swapping adapters into a
model, freezing everything else, and merging back."""

from __future__ import annotations

import math

import torch
import torch.nn as nn


class LowRankAdapter(nn.Module):
    """``linear`` plus a rank-``rank`` update ``B @ A`` scaled by ``lora_alpha / rank``.
    ``A`` is Kaiming-uniform, ``B`` zero, so a fresh adapter leaves the layer's output unchanged.
    ``rank == 0`` degenerates to the plain linear layer."""

    def __init__(self, in_features: int, out_features: int, rank: int = 0, lora_alpha: int = 1,
                 lora_dropout: float = 0.0, **kwargs) -> None:
        super().__init__()
        self.rank = rank
        self.lora_alpha = lora_alpha
        self.merged = False
        self.lora_dropout = nn.Dropout(p=lora_dropout) if lora_dropout > 0.0 else nn.Identity()
        self.linear = nn.Linear(in_features, out_features, **kwargs)
        if rank > 0:
            self.lora_A = nn.Parameter(torch.zeros((rank, in_features)))
            self.lora_B = nn.Parameter(torch.zeros((out_features, rank)))
            self.scaling = self.lora_alpha / self.rank
            self._register_extra_parameters(out_features)
            self.reset_parameters()

    # hooks for subclasses -------------------------------------------------------------------
    def _register_extra_parameters(self, out_features: int) -> None:
        pass

    def _reset_extra_parameters(self) -> None:
        pass

    def _adapter_parameters(self) -> list[nn.Parameter]:
        return [self.lora_A, self.lora_B]

    # shared behaviour -----------------------------------------------------------------------
    def delta(self) -> torch.Tensor:
        return (self.lora_B @ self.lora_A) * self.scaling

    def reset_adapter_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B)
        self._reset_extra_parameters()

    def reset_parameters(self, lora_only: bool = False) -> None:
        if not lora_only:
            nn.init.kaiming_normal_(self.linear.weight, a=math.sqrt(5))
        if self.rank > 0:
            self.reset_adapter_parameters()

    def adapter_trainable_only(self) -> None:
        self.linear.train(False)
        for p in self._adapter_parameters():
            p.requires_grad = True


def adapter_from_linear(cls, linear: nn.Linear, lora_alpha: int, lora_dropout: float, rank: int):
    """Build ``cls`` around a copy of ``linear``'s weights, on its device and dtype."""
    adapter = cls(linear.in_features, linear.out_features, lora_alpha=lora_alpha,
                  lora_dropout=lora_dropout, rank=rank, bias=linear.bias is not None)
    adapter = adapter.to(linear.weight.device)
    with torch.no_grad():
        adapter.linear.weight.copy_(linear.weight)
        if linear.bias is not None:
            adapter.linear.bias.copy_(linear.bias)
    if rank > 0:
        adapter._reset_extra_parameters()
    return adapter.to(linear.weight.dtype)


def replace_linears(cls, model: nn.Module, target_layer: list[str] | None, lora_alpha: int,
                    lora_dropout: float, rank: int):
    """Recursively replace ``nn.Linear`` children (all, or those named in ``target_layer``)."""
    if isinstance(model, nn.Linear):
        return adapter_from_linear(cls, model, lora_alpha, lora_dropout, rank)
    for name, child in model.named_children():
        if isinstance(child, nn.Linear) and (target_layer is None or name in target_layer):
            setattr(model, name, adapter_from_linear(cls, child, lora_alpha, lora_dropout, rank))
        else:
            replace_linears(cls, child, target_layer, lora_alpha, lora_dropout, rank)
    return model


def mark_only_adapters_trainable(cls, model: nn.Module) -> nn.Module:
    for p in model.parameters():
        p.requires_grad = False
    for module in model.modules():
        if isinstance(module, cls):
            module.adapter_trainable_only()
    return model


def merge_adapters(cls, model: nn.Module) -> nn.Module:
    for module in model.modules():
        if isinstance(module, cls):
            module.merge()
    return model
