"""BitNet b1.58 layers (reference: experiments/bitnet/bitnet.py:29-95).

Weights are quantised to {-1, 0, +1} times one scale per tensor (absolute-mean scaling),
activations to int8 per row (absolute-max scaling); both through straight-through estimators, so
the full-precision "shadow" weights keep receiving gradients. The quantisers and the layer's
function live in ``ohara_b200.ops.bitnet``; on a GPU the layer runs its kernels.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200.modules.norm import RMSNorm
from ohara_b200.ops.bitnet import activation_quant_reference as activation_quant
from ohara_b200.ops.bitnet import bit_linear
from ohara_b200.ops.bitnet import weight_quant_reference as weight_quant

__all__ = ["BitLinear", "activation_quant", "apply_bitlinear", "bit_linear", "weight_quant"]


class BitLinear(nn.Linear):
    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.rms_norm = RMSNorm(self.in_features)

    def forward(self, x: Tensor) -> Tensor:
        if x.is_cuda:  # quantiser kernels around the tensor-core GEMM, same gradients
            return bit_linear(x, self.weight, self.rms_norm.weight, self.bias, self.rms_norm.eps)
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
