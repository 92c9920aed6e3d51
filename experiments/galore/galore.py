"""AdamW with GaLore: Adam's moments of a matrix live in a rank-``r`` subspace of its gradient
(https://arxiv.org/abs/2403.03507; reference: experiments/galore/galore.py:14-238).

Parameter groups that carry ``rank`` project every 2-D gradient with a
:class:`experiments.misc.small_modules.GaLoreProjector` (refreshed from the gradient's SVD every
``update_proj_gap`` steps), run Adam in the projected space and project the normalised update back,
scaled by ``scale``. Optimizer state for an ``m x n`` matrix shrinks from ``2 m n`` to
``2 r max(m, n)`` numbers plus the ``r min(m, n)`` projector. Other groups are plain AdamW."""

from __future__ import annotations

import math
from typing import Callable, Iterable

import torch
from torch.optim import Optimizer

from experiments.misc.small_modules import GaLoreProjector


class GaLoreAdamW(Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-6, weight_decay: float = 0.0, correct_bias: bool = True) -> None:
        if lr < 0 or eps < 0 or not all(0.0 <= b < 1.0 for b in betas):
            raise ValueError("invalid AdamW hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      correct_bias=correct_bias))

    @torch.no_grad()
    def step(self, closure: Callable | None = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                state.setdefault("step", 0)
                grad = p.grad
                low_rank = "rank" in group and grad.ndim == 2
                if low_rank:
                    if "projector" not in state:
                        state["projector"] = GaLoreProjector(
                            group["rank"], update_gap=group.get("update_proj_gap", 200),
                            scale=group.get("scale", 1.0))
                    grad = state["projector"].project(grad, state["step"])
                if "exp_avg" not in state or state["exp_avg"].shape != grad.shape:
                    state["exp_avg"] = torch.zeros_like(grad)
                    state["exp_avg_sq"] = torch.zeros_like(grad)
                state["step"] += 1
                state["exp_avg"].mul_(beta1).add_(grad, alpha=1 - beta1)
                state["exp_avg_sq"].mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
                step_size = group["lr"]
                if group["correct_bias"]:
                    step_size *= math.sqrt(1 - beta2 ** state["step"]) / (1 - beta1 ** state["step"])
                update = state["exp_avg"] / state["exp_avg_sq"].sqrt().add_(group["eps"])
                if low_rank:
                    update = state["projector"].project_back(update)
                p.add_(update, alpha=-step_size)
                if group["weight_decay"] > 0:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
        return loss

    def state_numbers(self) -> int:
        """Numbers held in moments and projectors (what GaLore is meant to shrink)."""
        total = 0
        for state in self.state.values():
            total += state["exp_avg"].numel() + state["exp_avg_sq"].numel()
            projector = state.get("projector")
            if projector is not None and projector.basis is not None:
                total += projector.basis.numel()
        return total


def galore_param_groups(model: torch.nn.Module, rank: int, update_proj_gap: int = 200,
                        scale: float = 0.25, min_dim: int = 2) -> list[dict]:
    """Matrices of ``nn.Linear`` layers go to the low-rank group, everything else to plain AdamW."""
    low = [m.weight for m in model.modules()
           if isinstance(m, torch.nn.Linear) and min(m.weight.shape) > max(rank, min_dim)]
    low_ids = {id(p) for p in low}
    rest = [p for p in model.parameters() if id(p) not in low_ids]
    return [{"params": rest},
            {"params": low, "rank": rank, "update_proj_gap": update_proj_gap, "scale": scale}]
