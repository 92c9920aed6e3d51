"""Auxiliary objective on recurrent states: predict your own state ``n`` steps ahead
(reference: experiments/mihawk/state_shift.py:6-36)."""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor


def states_shift(states: Tensor, n: int) -> Tensor:
    """``out[:, t] = states[:, t + n]`` along dim 1, zeros where ``t + n`` runs off the end."""
    if n <= 0:
        return states
    n = min(n, states.shape[1])
    return torch.cat([states[:, n:], states.new_zeros(states.shape[0], n, *states.shape[2:])], dim=1)


def state_prediction_loss(states: Tensor, shift: int) -> Tensor:
    """Mean squared distance between a state and the state ``shift`` steps later; the last
    ``shift`` positions, which have no successor, contribute zero (they still count in the mean,
    as in the reference)."""
    valid = states_shift(torch.ones_like(states), shift)
    return F.mse_loss(states * valid, states_shift(states, shift))
