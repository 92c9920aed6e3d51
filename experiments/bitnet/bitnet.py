"""BitNet b1.58 layers (reference: experiments/bitnet/bitnet.py:29-95).

Weights are quantised to {-1, 0, +1} times one scale per tensor (absolute-mean scaling),
activations to int8 per row (absolute-max scaling); both through straight-through estimators, so
the full-precision "shadow" weights keep receiving gradients.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200.modules.norm import RMSNorm


def activation_quant(x: Tensor) -> Tensor:
    """Per-row int8 fake quantisation; the backward pass sees the identity."""
    scale = 127.0 / x.abs().amax(dim=-1, keepdim=True).clamp_min(1e-5)
    quantised = (x * scale).round().clamp(-128, 127) / scale
    return x + (quantised - x).detach()


def weight_quant(w: Tensor) -> tuple[Tensor, Tensor]:
    """Ternary fake quantisation. Returns the weight normalised to {-1, 0, 1} (with the
    straight-through gradient of ``w``) and the scale to multiply the product by."""
    inv = 1.0 / w.abs().mean().clamp_min(1e-5)
    ternary = (w * inv).round().clamp(-1, 1) / inv
    w_ste = w + (ternary - w).detach()
    scale = w_ste.abs().max().detach()
    return w_ste / scale, scale


class BitLinear(nn.Linear):
    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.rms_norm = RMSNorm(self.in_features)

    def forward(self, x: Tensor) -> Tensor:
        w, scale = weight_quant(self.weight)
        out = F.linear(activation_quant(self.rms_norm(x)), w) * scale
        return out if self.bias is None else out + self.bias


def apply_bitlinear(model: nn.Module, target_layers: list[str] | None = None) -> nn.Module:
    """Replace ``nn.Linear`` children (all, or those whose attribute name is listed) in place."""
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear) and not isinstance(child, BitLinear) and (
                target_layers is None or name in target_layers):
            layer = BitLinear(child.in_features, child.out_features, bias=child.bias is not None)
            layer.to(device=child.weight.device, dtype=child.weight.dtype)
            with torch.no_grad():
                layer.weight.copy_(child.weight)
                if child.bias is not None:
                    layer.bias.copy_(child.bias)
            setattr(model, name, layer)
        else:
            apply_bitlinear(child, target_layers)
    return model
