"""RMSNorm (https://arxiv.org/abs/1910.07467).

Semantics of the reference (ohara/modules/norm.py:7-24): normalise in fp32, cast back to the input
dtype, then scale by the learned gain. On CUDA the whole thing is one fused kernel per direction.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor


def rms_norm_reference(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    xf = x.float()
    normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x)
    return normed * weight


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: Tensor) -> Tensor:
        if x.is_cuda:
            from ohara_b200.ops import rms_norm

            return rms_norm(x, self.weight, self.eps)
        return rms_norm_reference(x, self.weight, self.eps)

    def reset_parameters(self) -> None:
        nn.init.ones_(self.weight)
