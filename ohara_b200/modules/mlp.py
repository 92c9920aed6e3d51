"""Feed-forward blocks: plain MLP and the gated-linear-unit family (https://arxiv.org/abs/2002.05202).

Attribute names (`up`, `gate`, `down`, `w1..w3`) follow the reference so state dicts interchange
(ohara/modules/mlp.py:10-281). Linear layers go through :func:`ohara_b200.ops.linear`, so on a CUDA
device inside bf16 autocast the projections run on the tcgen05 GEMM and SwiGLU's activation is one
fused kernel.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200 import ops
from ohara_b200.modules.activations import ACT2FN  # noqa: F401  (re-exported)


def default_hidden_dim(dim: int, multiple_of: int = 4) -> int:
    """``8/3 * dim`` rounded up to ``multiple_of`` — the LLaMA feed-forward width rule."""
    hidden = int(2 * (4 * dim) / 3)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


class Linear(nn.Linear):
    """``nn.Linear`` whose forward dispatches to the sm_100a GEMM on the bf16 fast path."""

    def forward(self, x: Tensor) -> Tensor:  # noqa: D401
        return ops.linear(x, self.weight, self.bias)


def _dropout(p: float | None):
    return nn.Dropout(p) if p else nn.Identity()


def _trunc_normal(weight: Tensor, std: float) -> None:
    nn.init.trunc_normal_(weight, mean=0.0, std=std, a=-3 * std, b=3 * std)


class _FeedForward(nn.Module):
    dim: int
    hidden_dim: int

    def _init_in_out(self, in_layers, out_layer, init_std=None, factor: float = 1.0) -> None:
        in_std = init_std or self.dim**-0.5
        out_std = (init_std or self.hidden_dim**-0.5) / factor
        for layer in in_layers:
            _trunc_normal(layer.weight, in_std)
        _trunc_normal(out_layer.weight, out_std)


class MLP(_FeedForward):
    def __init__(self, dim: int, hidden_dim: int | None = None, multiple_of: int = 4,
                 dropout: float | None = None, activation_fn: str = "silu", bias: bool = True):
        super().__init__()
        self.dim = dim
        self.hidden_dim = hidden_dim or default_hidden_dim(dim, multiple_of)
        self.up = Linear(dim, self.hidden_dim, bias=bias)
        self.down = Linear(self.hidden_dim, dim, bias=bias)
        self.activation_fn = ACT2FN[activation_fn]
        self.dropout = _dropout(dropout)

    def forward(self, x: Tensor) -> Tensor:
        return self.dropout(self.down(self.activation_fn(self.up(x))))

    def reset_parameters(self, init_std=None, factor: float = 1.0) -> None:
        self._init_in_out([self.up], self.down, init_std, factor)


class GLU(_FeedForward):
    """Generic gated unit ``down(act(gate(x)) * up(x))`` with a selectable activation."""

    def __init__(self, dim: int, hidden_dim: int | None = None, multiple_of: int = 4,
                 dropout: float | None = None, activation_fn: str = "silu", bias: bool = False,
                 *args, **kwargs):
        super().__init__()
        self.dim = dim
        self.hidden_dim = hidden_dim or default_hidden_dim(dim, multiple_of)
        # (created in the reference's order, up / gate / down, so that the same seed gives the
        # same initial weights: ohara/modules/mlp.py:90-92; SwiGLU's order is up / down / gate)
        self.up = Linear(dim, self.hidden_dim, bias=bias)
        self.gate = Linear(dim, self.hidden_dim, bias=bias)
        self.down = Linear(self.hidden_dim, dim, bias=bias)
        self.activation = ACT2FN[activation_fn]
        self.dropout = _dropout(dropout)

    def forward(self, x: Tensor) -> Tensor:
        return self.dropout(self.down(self.activation(self.gate(x)) * self.up(x)))

    def reset_parameters(self, init_std=None, factor: float = 1.0) -> None:
        self._init_in_out([self.up, self.gate], self.down, init_std, factor)


class SwiGLU(_FeedForward):
    def __init__(self, dim: int, hidden_dim: int | None = None, multiple_of: int = 4,
                 dropout: float | None = None, bias: bool = False):
        super().__init__()
        self.dim = dim
        self.hidden_dim = hidden_dim or default_hidden_dim(dim, multiple_of)
        self.up = Linear(dim, self.hidden_dim, bias=bias)
        self.down = Linear(self.hidden_dim, dim, bias=bias)
        self.gate = Linear(dim, self.hidden_dim, bias=bias)
        self.dropout = _dropout(dropout)

    def forward(self, x: Tensor) -> Tensor:
        plain = (type(self.gate) is Linear and type(self.up) is Linear and self.gate.bias is None
                 and self.up.bias is None)
        if plain and ops.fused_projections(x) and self.hidden_dim % 8 == 0:
            # one gate|up GEMM; the activation reads its two halves and returns one gradient
            fused = ops.linear_cat(x, (self.gate.weight, self.up.weight))
            return self.dropout(self.down(ops.swiglu_cat(fused)))
        if not plain and self.hidden_dim % 8 == 0:
            from ohara_b200.runtime.tensor_parallel import ColumnParallelLinear, fused_column_parallel

            if type(self.gate) is ColumnParallelLinear and (self.gate.weight.shape[0] % 8 == 0):
                fused = fused_column_parallel(x, (self.gate, self.up))
                if fused is not None:  # one gather + one GEMM for this rank's gate | up columns
                    return self.dropout(self.down(ops.swiglu_cat(fused)))
        if plain:
            gate, up = ops.linear_fanout(x, (self.gate.weight, self.up.weight))
        else:  # biases, adapters or tensor-parallel replacements
            gate, up = self.gate(x), self.up(x)
        return self.dropout(self.down(ops.swiglu(gate, up)))

    def reset_parameters(self, init_std=None, factor: float = 1.0) -> None:
        self._init_in_out([self.up, self.gate], self.down, init_std, factor)


class _W123(_FeedForward):
    def __init__(self, dim: int, hidden_dim: int | None = None, multiple_of: int = 4,
                 dropout: float | None = None, bias: bool = False):
        super().__init__()
        self.dim = dim
        self.hidden_dim = hidden_dim or default_hidden_dim(dim, multiple_of)
        self.w1 = Linear(dim, self.hidden_dim, bias=bias)
        self.w2 = Linear(self.hidden_dim, dim, bias=bias)
        self.w3 = Linear(dim, self.hidden_dim, bias=bias)
        self.dropout = _dropout(dropout)


class BiLinear(_W123):
    def forward(self, x: Tensor) -> Tensor:
        return self.dropout(self.w2(self.w1(x) * self.w3(x)))


class ReGLU(_W123):
    def forward(self, x: Tensor) -> Tensor:
        return self.dropout(self.w2(F.relu(self.w1(x)) * self.w3(x)))


class GEGLU(_FeedForward):
    def __init__(self, dim: int, hidden_dim: int | None = None, multiple_of: int = 4,
                 dropout: float | None = None, bias: bool = False):
        super().__init__()
        self.dim = dim
        self.hidden_dim = hidden_dim or default_hidden_dim(dim, multiple_of)
        self.gate = Linear(dim, self.hidden_dim, bias=bias)
        self.up = Linear(dim, self.hidden_dim, bias=bias)
        self.down = Linear(self.hidden_dim, dim, bias=bias)
        self.dropout = _dropout(dropout)

    def forward(self, x: Tensor) -> Tensor:
        return self.dropout(self.down(F.gelu(self.gate(x)) * self.up(x)))


MLP_MAP = {
    "swiglu": SwiGLU,
    "mlp": MLP,
    "glu": GLU,
    "bilinear": BiLinear,
    "reglu": ReGLU,
    "geglu": GEGLU,
}
