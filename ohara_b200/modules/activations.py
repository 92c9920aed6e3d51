"""Name → activation registry (reference: ohara/modules/activations.py:5-17)."""

import torch
import torch.nn.functional as F


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    return torch.relu(x).square()


ACT2FN = {
    "relu": F.relu,
    "silu": F.silu,
    "gelu": F.gelu,
    "tanh": torch.tanh,
    "sigmoid": torch.sigmoid,
    "relu_squared": relu_squared,
    "relu2": relu_squared,
}
