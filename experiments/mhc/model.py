"""A small language model whose blocks are joined by residual, hyper- or manifold-constrained
hyper-connections (reference: experiments/mHC/model.py:23-434).

``connection_type``:

* ``"residual"``: ``x + f(norm(x))``;
* ``"mhc"``: ``rate`` parallel streams; every sub-layer reads a learned mix of them and writes
  back through a doubly stochastic stream-mixing matrix (Sinkhorn projection:
  :func:`ohara_b200.ops.sinkhorn.sinkhorn_log`, CUDA kernels for up to 64 streams);
* ``"hc"``: the same without the projection (the mixing matrix is used as predicted, plus the
  identity), the unconstrained baseline the manifold constraint is compared with.

The streams start as copies of the embedding and are averaged before the final norm."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
from torch import Tensor

from experiments.mhc.hyper_connections import ManifoldHyperConnections
from ohara_b200.embeddings_pos.rotary import precompute_freqs_cis
from ohara_b200.modules.mlp import SwiGLU
from ohara_b200.modules.norm import RMSNorm
from experiments.partial_kv.pkv import FullAttention


@dataclass
class MHCConfig:
    vocab_size: int = 256
    max_sequence_length: int = 256
    hidden_size: int = 128
    intermediate_size: int = 256
    num_attention_heads: int = 4
    num_hidden_layers: int = 4
    expansion_rate: int = 4
    connection_type: str = "mhc"  # "residual", "hc", "mhc"
    mhc_sinkhorn_iters: int = 20
    dropout: float = 0.0


class _Connected(nn.Module):
    """One sub-layer ``f`` (``(b, t, d) -> (b, t, d)``) behind the chosen kind of connection."""

    def __init__(self, layer: nn.Module, cfg: MHCConfig) -> None:
        super().__init__()
        self.layer, self.kind = layer, cfg.connection_type
        self.norm = RMSNorm(cfg.hidden_size)
        if self.kind not in ("residual", "hc", "mhc"):
            raise ValueError(f"unknown connection_type {self.kind!r}")
        if self.kind != "residual":
            self.connections = ManifoldHyperConnections(cfg.hidden_size, cfg.expansion_rate,
                                                        cfg.mhc_sinkhorn_iters)

    def _mixing(self, streams: Tensor):
        connections = self.connections
        if self.kind == "mhc":
            return connections(streams)
        # unconstrained: the raw prediction plus the identity instead of the Sinkhorn projection
        pre, post, res = connections.raw_mixing(streams)
        identity = torch.eye(streams.shape[2], device=res.device)
        return torch.sigmoid(pre), 2.0 * torch.sigmoid(post), res + identity

    def forward(self, streams: Tensor, *args) -> Tensor:
        if self.kind == "residual":
            return streams + self.layer(self.norm(streams), *args)
        h_pre, h_post, h_res = self._mixing(streams)
        layer_in = (h_pre.unsqueeze(-1) * streams).sum(dim=2)
        layer_out = self.layer(self.norm(layer_in), *args)
        return torch.einsum("btji,btid->btjd", h_res, streams) + h_post.unsqueeze(-1) * layer_out.unsqueeze(2)


class MHCModel(nn.Module):
    def __init__(self, cfg: MHCConfig) -> None:
        super().__init__()
        self.config = cfg
        self.token_emb = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.attention = nn.ModuleList(
            _Connected(FullAttention(cfg.hidden_size, cfg.num_attention_heads, cfg.dropout), cfg)
            for _ in range(cfg.num_hidden_layers))
        self.feed_forward = nn.ModuleList(
            _Connected(SwiGLU(cfg.hidden_size, cfg.intermediate_size), cfg)
            for _ in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size)
        self.vocab_proj = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        cos, sin = precompute_freqs_cis(cfg.hidden_size // cfg.num_attention_heads,
                                        cfg.max_sequence_length)
        self.register_buffer("freq_cos", cos, persistent=False)
        self.register_buffer("freq_sin", sin, persistent=False)

    def forward(self, tokens: Tensor) -> Tensor:
        steps = tokens.shape[1]
        freqs = (self.freq_cos[:steps], self.freq_sin[:steps])
        x = self.token_emb(tokens)
        wide = self.config.connection_type != "residual"
        if wide:
            x = x.unsqueeze(2).expand(-1, -1, self.config.expansion_rate, -1).contiguous()
        for attention, feed_forward in zip(self.attention, self.feed_forward):
            x = attention(x, freqs)
            x = feed_forward(x)
        if wide:
            x = x.mean(dim=2)
        return self.vocab_proj(self.norm(x))
