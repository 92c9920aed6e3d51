"""Preference-optimisation losses from sequence log-probabilities: DPO
(https://arxiv.org/abs/2305.18290), conservative DPO with label smoothing, and IPO. Reference:
ohara/dpo.py:9-178.

With ``h = (log π(win) − log π(lose)) − (log ref(win) − log ref(lose))``:
DPO ``−log σ(βh)``; cDPO ``−(1−ε) log σ(βh) − ε log σ(−βh)``; IPO ``(h − 1/(2β))²``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

IGNORE_INDEX = -100


def sequence_logps(logits: Tensor, labels: Tensor, ignore_index: int = IGNORE_INDEX) -> Tensor:
    """Summed log-probability of ``labels (B, T)`` under ``logits (B, T, V)``, skipping masked
    positions; returns ``(B,)``."""
    keep = labels != ignore_index
    picked = F.log_softmax(logits, dim=-1).gather(-1, labels.masked_fill(~keep, 0).unsqueeze(-1))
    return (picked.squeeze(-1) * keep).sum(dim=-1)


def _margin(pi_win: Tensor, pi_lose: Tensor, ref_win: Tensor, ref_lose: Tensor) -> Tensor:
    return (pi_win - pi_lose) - (ref_win - ref_lose)


def _pair_rewards(pi_win, pi_lose, ref_win, ref_lose, beta: float) -> Tensor:
    return beta * (torch.stack([pi_win, pi_lose]) - torch.stack([ref_win, ref_lose])).detach()


def dpo_loss_from_logps(pi_win_logps: Tensor, pi_lose_logps: Tensor, ref_win_logps: Tensor,
                        ref_lose_logps: Tensor, beta: float) -> tuple[Tensor, Tensor]:
    h = _margin(pi_win_logps, pi_lose_logps, ref_win_logps, ref_lose_logps)
    return -F.logsigmoid(beta * h), _pair_rewards(pi_win_logps, pi_lose_logps, ref_win_logps,
                                                  ref_lose_logps, beta)


def cdpo_loss_from_logps(pi_win_logps: Tensor, pi_lose_logps: Tensor, ref_win_logps: Tensor,
                         ref_lose_logps: Tensor, beta: float,
                         label_smoothing: float = 0.2) -> tuple[Tensor, Tensor]:
    h = _margin(pi_win_logps, pi_lose_logps, ref_win_logps, ref_lose_logps)
    losses = (-F.logsigmoid(beta * h) * (1 - label_smoothing)
              - F.logsigmoid(-beta * h) * label_smoothing)
    return losses, _pair_rewards(pi_win_logps, pi_lose_logps, ref_win_logps, ref_lose_logps, beta)


def ipo_loss_from_logps(pi_win_logps: Tensor, pi_lose_logps: Tensor, ref_win_logps: Tensor,
                        ref_lose_logps: Tensor, beta: float) -> tuple[Tensor, Tensor]:
    h = _margin(pi_win_logps, pi_lose_logps, ref_win_logps, ref_lose_logps)
    return (h - 1 / (2 * beta)) ** 2, _pair_rewards(pi_win_logps, pi_lose_logps, ref_win_logps,
                                                    ref_lose_logps, beta)


def _indexed(fn, pi_logps, ref_logps, win_idx, lose_idx, beta, **extra):
    losses, _ = fn(pi_logps[win_idx], pi_logps[lose_idx], ref_logps[win_idx], ref_logps[lose_idx],
                   beta, **extra)
    return losses, beta * (pi_logps - ref_logps).detach()


def dpo_loss(pi_logps: Tensor, ref_logps: Tensor, win_output_idxs: Tensor,
             lose_output_idxs: Tensor, beta: float) -> tuple[Tensor, Tensor]:
    """Index-based wrapper: ``pi_logps`` / ``ref_logps`` hold all sequences of a batch; the index
    tensors pick the preferred and rejected ones. Rewards cover every sequence."""
    return _indexed(dpo_loss_from_logps, pi_logps, ref_logps, win_output_idxs, lose_output_idxs, beta)


def cdpo_loss(pi_logps: Tensor, ref_logps: Tensor, win_output_idxs: Tensor,
              lose_output_idxs: Tensor, beta: float, label_smoothing=0.2) -> tuple[Tensor, Tensor]:
    return _indexed(cdpo_loss_from_logps, pi_logps, ref_logps, win_output_idxs, lose_output_idxs,
                    beta, label_smoothing=label_smoothing)


def ipo_loss(pi_logps: Tensor, ref_logps: Tensor, win_output_idxs: Tensor,
             lose_output_idxs: Tensor, beta: float) -> tuple[Tensor, Tensor]:
    return _indexed(ipo_loss_from_logps, pi_logps, ref_logps, win_output_idxs, lose_output_idxs, beta)
