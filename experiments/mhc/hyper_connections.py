"""Manifold-constrained hyper-connections (reference: experiments/mHC/model.py:56-105).

The residual stream is widened to ``rate`` parallel streams. For every token three small mixing
objects are predicted from the (RMS-normalised, flattened) streams: ``h_pre`` (how the streams are
combined into the layer input, sigmoid gates), ``h_post`` (how the layer output is written back,
``2 * sigmoid``) and ``h_res`` (a ``rate x rate`` stream-mixing matrix projected onto the doubly
stochastic matrices with Sinkhorn iterations, which keeps the residual path norm-preserving).
The Sinkhorn projection is ``ohara_b200.ops.sinkhorn.sinkhorn_log`` (a CUDA kernel for
``rate <= 4`` on a GPU).
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200.modules.norm import RMSNorm
from ohara_b200.ops.sinkhorn import sinkhorn_log


class ManifoldHyperConnections(nn.Module):
    def __init__(self, dim: int, rate: int, sinkhorn_iters: int = 20) -> None:
        super().__init__()
        self.dim, self.rate, self.sinkhorn_iters = dim, rate, sinkhorn_iters
        flat = dim * rate
        self.norm = RMSNorm(flat)
        # (parameter names and shapes are the reference's, so its state dicts load here)
        self.phi_pre = nn.Parameter(torch.zeros(flat, rate))
        self.phi_post = nn.Parameter(torch.zeros(flat, rate))
        self.phi_res = nn.Parameter(torch.zeros(flat, rate * rate))
        self.b_pre = nn.Parameter(torch.zeros(rate))
        self.b_post = nn.Parameter(torch.zeros(rate))
        self.b_res = nn.Parameter(torch.zeros(rate, rate))
        self.alpha_pre = nn.Parameter(torch.full((1,), 0.01))  # small gates at initialisation
        self.alpha_post = nn.Parameter(torch.full((1,), 0.01))
        self.alpha_res = nn.Parameter(torch.full((1,), 0.01))

    def raw_mixing(self, streams: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        """The three predictions before their squashing functions: ``pre`` and ``post``
        ``(b, t, rate)``, ``res`` ``(b, t, rate, rate)``."""
        b, t, r, _ = streams.shape
        # one product for the three projections
        proj = self.norm(streams.flatten(2)) @ torch.cat((self.phi_pre, self.phi_post, self.phi_res), dim=1)
        pre = self.alpha_pre * proj[..., :r] + self.b_pre
        post = self.alpha_post * proj[..., r:2 * r] + self.b_post
        res = (self.alpha_res * proj[..., 2 * r:]).view(b, t, r, r) + self.b_res
        return pre, post, res

    def forward(self, streams: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        """``streams``: (batch, seq, rate, dim) -> ``h_pre`` (b, t, rate), ``h_post`` (b, t, rate),
        ``h_res`` (b, t, rate, rate)."""
        pre, post, res = self.raw_mixing(streams)
        return torch.sigmoid(pre), 2.0 * torch.sigmoid(post), sinkhorn_log(res, self.sinkhorn_iters)


class HyperConnectedBlock(nn.Module):
    """Wraps a ``(batch, seq, dim) -> (batch, seq, dim)`` layer with hyper-connections:
    ``x_in = sum_i h_pre_i * stream_i``; ``stream_j <- sum_i h_res_ji * stream_i + h_post_j * f(x_in)``."""

    def __init__(self, layer: nn.Module, dim: int, rate: int, sinkhorn_iters: int = 20) -> None:
        super().__init__()
        self.layer = layer
        self.connections = ManifoldHyperConnections(dim, rate, sinkhorn_iters)

    def forward(self, streams: Tensor) -> Tensor:
        h_pre, h_post, h_res = self.connections(streams)
        layer_in = (h_pre.unsqueeze(-1) * streams).sum(dim=2)
        layer_out = self.layer(layer_in)
        mixed = torch.einsum("btji,btid->btjd", h_res, streams)
        return mixed + h_post.unsqueeze(-1) * layer_out.unsqueeze(2)
