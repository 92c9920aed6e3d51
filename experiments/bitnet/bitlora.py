"""Low-rank adapters on ternary layers (reference: experiments/bitnet/bitlora.py:16-83).

``BitLora`` adds ``scaling * (A @ B)^T`` to the full-precision shadow weight *before* the ternary
quantisation, so the adapted layer is still a ternary layer at inference time; ``merge`` folds the
adapter into the shadow weight. (The reference adds ``A @ B`` with shape ``(in, out)`` to a weight
of shape ``(out, in)``, which only runs for square layers, and merges ``B @ A``, a ``rank x rank``
matrix; here the product is laid out as the weight.) ``B`` starts at zero, so a fresh adapter
leaves the layer unchanged."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from experiments.bitnet.bitnet import BitLinear, activation_quant, weight_quant


class BitLora(BitLinear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, rank: int = 4,
                 lora_alpha: float = 1.0) -> None:
        super().__init__(in_features, out_features, bias=bias)
        self.rank, self.scaling, self.merged = rank, lora_alpha / max(rank, 1), False
        self.lora_A = nn.Parameter(torch.randn(rank, in_features) * in_features**-0.5)
        self.lora_B = nn.Parameter(torch.zeros(out_features, rank))

    def adapted_weight(self) -> Tensor:
        if self.merged or self.rank == 0:
            return self.weight
        return self.weight + self.scaling * (self.lora_B @ self.lora_A)

    def forward(self, x: Tensor) -> Tensor:
        w, scale = weight_quant(self.adapted_weight())
        out = F.linear(activation_quant(self.rms_norm(x)), w) * scale
        return out if self.bias is None else out + self.bias

    @torch.no_grad()
    def merge(self) -> None:
        if not self.merged and self.rank > 0:
            self.weight.add_(self.scaling * (self.lora_B @ self.lora_A))
            self.merged = True


def apply_bitlora(model: nn.Module, target_layers: list[str] | None = None, rank: int = 4,
                  lora_alpha: float = 1.0, train_base: bool = False) -> nn.Module:
    """Replace linear layers (all, or those whose attribute name is listed) by ``BitLora`` copies;
    only the adapters stay trainable unless ``train_base``."""
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear) and not isinstance(child, BitLora) and (
                target_layers is None or name in target_layers):
            layer = BitLora(child.in_features, child.out_features, child.bias is not None, rank,
                            lora_alpha).to(child.weight.device, child.weight.dtype)
            with torch.no_grad():
                layer.weight.copy_(child.weight)
                if child.bias is not None:
                    layer.bias.copy_(child.bias)
            setattr(model, name, layer)
        else:
            apply_bitlora(child, target_layers, rank, lora_alpha, train_base)
    if not train_base:
        for name, parameter in model.named_parameters():
            parameter.requires_grad_("lora_" in name)
    return model
