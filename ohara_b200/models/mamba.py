"""Mamba (selective state-space model, https://arxiv.org/abs/2312.00752).

Block: ``in_proj`` → (x, z); depthwise causal ``conv1d`` + SiLU on x; input-dependent
``Δ, B, C = x_proj(x)`` with ``Δ = softplus(dt_proj(·))``; discretised diagonal SSM
``h_t = exp(Δ_t A) h_{t-1} + Δ_t B_t x_t``, ``y_t = C_t h_t + D x_t``; gate by SiLU(z);
``out_proj``. Training uses the parallel scan of :mod:`ohara_b200.modules.pscan` (or a
sequential loop when ``config.pscan`` is off); ``step`` is the O(1)-per-token recurrent form with
a (state, conv window) cache. Module and parameter names follow the reference
(ohara/models/mamba.py:58-412) so state dicts interchange.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200.modules.norm import RMSNorm
from ohara_b200.modules.pscan import pscan


@dataclass
class MambaConfig:
    d_model: int
    n_layers: int
    dt_rank: int | str = "auto"
    d_state: int = 16
    expand_factor: int = 2
    d_conv: int = 4
    dt_min: float = 0.001
    dt_max: float = 0.1
    dt_init: str = "random"  # or "constant"
    dt_scale: float = 1.0
    dt_init_floor = 1e-4
    bias: bool = False
    conv_bias: bool = True
    pscan: bool = True

    def __post_init__(self):
        self.d_inner = self.expand_factor * self.d_model
        if self.dt_rank == "auto":
            self.dt_rank = math.ceil(self.d_model / 16)


class Mamba(nn.Module):
    """Stack of residual Mamba blocks over ``(B, L, D)`` activations (no embedding / head)."""

    def __init__(self, config: MambaConfig):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([ResidualBlock(config) for _ in range(config.n_layers)])

    def forward(self, x: Tensor) -> Tensor:
        for layer in self.layers:
            x = layer(x)
        return x

    def init_caches(self, batch_size: int, device=None, dtype=None) -> list:
        cfg = self.config
        return [
            (torch.zeros(batch_size, cfg.d_inner, cfg.d_state, device=device, dtype=dtype),
             torch.zeros(batch_size, cfg.d_inner, cfg.d_conv - 1, device=device, dtype=dtype))
            for _ in self.layers
        ]

    def step(self, x: Tensor, caches: list):
        """One token ``(B, D)`` through every layer; ``caches[i] = (h, conv_inputs)``."""
        for i, layer in enumerate(self.layers):
            x, caches[i] = layer.step(x, caches[i])
        return x, caches


class ResidualBlock(nn.Module):
    def __init__(self, config: MambaConfig):
        super().__init__()
        self.mixer = MambaBlock(config)
        self.norm = RMSNorm(config.d_model)

    def forward(self, x: Tensor) -> Tensor:
        return self.mixer(self.norm(x)) + x

    def step(self, x: Tensor, cache):
        out, cache = self.mixer.step(self.norm(x), cache)
        return out + x, cache


class MambaBlock(nn.Module):
    def __init__(self, config: MambaConfig):
        super().__init__()
        self.config = config
        inner, state, rank = config.d_inner, config.d_state, config.dt_rank
        self.in_proj = nn.Linear(config.d_model, 2 * inner, bias=config.bias)
        self.conv1d = nn.Conv1d(inner, inner, kernel_size=config.d_conv, bias=config.conv_bias,
                                groups=inner, padding=config.d_conv - 1)
        self.x_proj = nn.Linear(inner, rank + 2 * state, bias=False)
        self.dt_proj = nn.Linear(rank, inner, bias=True)
        # Δ projection init keeps softplus(bias) inside [dt_min, dt_max].
        std = rank**-0.5 * config.dt_scale
        if config.dt_init == "constant":
            nn.init.constant_(self.dt_proj.weight, std)
        elif config.dt_init == "random":
            nn.init.uniform_(self.dt_proj.weight, -std, std)
        else:
            raise NotImplementedError(f"unknown dt_init {config.dt_init!r}")
        dt = torch.exp(
            torch.rand(inner) * (math.log(config.dt_max) - math.log(config.dt_min))
            + math.log(config.dt_min)
        ).clamp(min=config.dt_init_floor)
        with torch.no_grad():
            self.dt_proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus
        # S4D-real initialisation: A = -(1..N) for every channel, stored as log.
        self.A_log = nn.Parameter(torch.log(torch.arange(1, state + 1, dtype=torch.float32).repeat(inner, 1)))
        self.D = nn.Parameter(torch.ones(inner))
        self.out_proj = nn.Linear(inner, config.d_model, bias=config.bias)

    # -- training / prefill ----------------------------------------------------------------------
    def forward(self, x: Tensor) -> Tensor:
        length = x.shape[1]
        branch, gate = self.in_proj(x).chunk(2, dim=-1)
        branch = F.silu(self.conv1d(branch.transpose(1, 2))[:, :, :length].transpose(1, 2))
        return self.out_proj(self.ssm(branch) * F.silu(gate))

    def _ssm_inputs(self, x: Tensor):
        cfg = self.config
        A = -torch.exp(self.A_log.float())
        delta, B, C = torch.split(self.x_proj(x), [cfg.dt_rank, cfg.d_state, cfg.d_state], dim=-1)
        return A, F.softplus(self.dt_proj(delta)), B, C

    def ssm(self, x: Tensor) -> Tensor:
        A, delta, B, C = self._ssm_inputs(x)
        scan = self.selective_scan if self.config.pscan else self.selective_scan_seq
        return scan(x, delta, A, B, C, self.D.float())

    @staticmethod
    def _discretise(x, delta, A, B):
        decay = torch.exp(delta.unsqueeze(-1) * A)  # (B, L, ED, N)
        drive = delta.unsqueeze(-1) * B.unsqueeze(2) * x.unsqueeze(-1)
        return decay, drive

    def selective_scan(self, x, delta, A, B, C, D):
        decay, drive = self._discretise(x, delta, A, B)
        states = pscan(decay, drive)
        return (states @ C.unsqueeze(-1)).squeeze(-1) + D * x

    def selective_scan_seq(self, x, delta, A, B, C, D):
        decay, drive = self._discretise(x, delta, A, B)
        h = torch.zeros_like(drive[:, 0])
        states = []
        for t in range(x.shape[1]):
            h = decay[:, t] * h + drive[:, t]
            states.append(h)
        states = torch.stack(states, dim=1)
        return (states @ C.unsqueeze(-1)).squeeze(-1) + D * x

    # -- recurrent inference ---------------------------------------------------------------------
    def step(self, x: Tensor, cache):
        """``x (B, D)``, ``cache = (h (B, ED, N) | None, window (B, ED, d_conv-1))``."""
        h, window = cache
        branch, gate = self.in_proj(x).chunk(2, dim=1)
        taps = torch.cat([window, branch.unsqueeze(-1)], dim=2)  # (B, ED, d_conv)
        conv = (taps * self.conv1d.weight.squeeze(1)).sum(-1)
        if self.conv1d.bias is not None:
            conv = conv + self.conv1d.bias
        y, h = self.ssm_step(F.silu(conv), h)
        return self.out_proj(y * F.silu(gate)), (h, taps[:, :, 1:])

    def ssm_step(self, x: Tensor, h: Tensor | None):
        cfg = self.config
        A = -torch.exp(self.A_log.float())
        delta, B, C = torch.split(self.x_proj(x), [cfg.dt_rank, cfg.d_state, cfg.d_state], dim=-1)
        delta = F.softplus(self.dt_proj(delta))
        decay = torch.exp(delta.unsqueeze(-1) * A)
        drive = delta.unsqueeze(-1) * B.unsqueeze(1) * x.unsqueeze(-1)
        if h is None:
            h = torch.zeros_like(drive)
        h = decay * h + drive
        return (h @ C.unsqueeze(-1)).squeeze(2) + self.D.float() * x, h
