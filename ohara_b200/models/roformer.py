"""RoFormer: the GPT layout with rotary position embeddings instead of learned ones and a GELU
MLP (https://arxiv.org/abs/2104.09864). Reference: ohara/models/roformer.py:22-160."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ohara_b200.embeddings_pos.rotary import precompute_freqs_cis
from ohara_b200.modules.mlp import MLP, Linear

from ._blocks import SelfAttention, check_token_ids


@dataclass
class Config:
    vocab_size: int = 65
    seq_len: int = 64
    d_model: int = 128
    num_heads: int = 4
    num_layers: int = 4
    dropout: float = 0.2
    multiple_of: int = 4
    bias: bool = True


class Attention(SelfAttention):
    def __init__(self, config: Config):
        super().__init__(config.d_model, config.num_heads, bias=config.bias, dropout=config.dropout)

    def forward(self, x, freqs_cis, mask=None):
        return super().forward(x, freqs_cis)


class Block(nn.Module):
    def __init__(self, config: Config):
        super().__init__()
        self.attn = Attention(config)
        self.ff = MLP(dim=config.d_model, multiple_of=config.multiple_of, dropout=config.dropout,
                      activation_fn="gelu", bias=config.bias)
        self.norm1 = nn.LayerNorm(config.d_model)
        self.norm2 = nn.LayerNorm(config.d_model)

    def forward(self, x, freqs_cis, mask=None):
        x = x + self.attn(self.norm1(x), freqs_cis, mask)
        return x + self.ff(self.norm2(x))


class RoFormer(nn.Module):
    def __init__(self, config: Config) -> None:
        super().__init__()
        if config.d_model % config.num_heads != 0:
            raise ValueError("d_model must be divisible by num_heads")
        head_dim = config.d_model // config.num_heads
        if head_dim % 2 != 0:
            raise ValueError("attention head dimension must be even for rotary embeddings")
        self.config = config
        self.word_emb = nn.Embedding(config.vocab_size, config.d_model)
        self.layers = nn.ModuleList([Block(config) for _ in range(config.num_layers)])
        self.norm = nn.LayerNorm(config.d_model)
        self.vocab_proj = Linear(config.d_model, config.vocab_size, bias=False)
        cos, sin = precompute_freqs_cis(head_dim, config.seq_len * 2)
        self.register_buffer("freq_cos", cos, persistent=False)
        self.register_buffer("freq_sin", sin, persistent=False)
        self.mask = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        seq = check_token_ids(x, self.config.seq_len)
        freqs = (self.freq_cos[:seq], self.freq_sin[:seq])
        h = self.word_emb(x)
        for layer in self.layers:
            h = layer(h, freqs, self.mask)
        return self.vocab_proj(self.norm(h))
