"""Minimal GPT: learned position embeddings, LayerNorm, causal MHA, selectable feed-forward
(``mlp`` is any key of ``MLP_MAP``). Reference: ohara/models/gpt.py:19-145."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ohara_b200.modules.mlp import MLP_MAP, Linear

from ._blocks import SelfAttention, check_token_ids


@dataclass
class Config:
    vocab_size: int = 65
    max_sequence_length: int = 64
    hidden_size: int = 128
    num_attention_heads: int = 4
    num_hidden_layers: int = 4
    dropout: float = 0.2
    multiple_of: int = 4
    bias: bool = False
    mlp: str = "mlp"


class Attention(SelfAttention):
    def __init__(self, config: Config):
        super().__init__(config.hidden_size, config.num_attention_heads, bias=config.bias,
                         dropout=config.dropout)
        self.num_attention_heads = config.num_attention_heads

    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
        return super().forward(x)


class Block(nn.Module):
    def __init__(self, config: Config):
        super().__init__()
        self.attn = Attention(config)
        self.ff = MLP_MAP[config.mlp](dim=config.hidden_size, multiple_of=config.multiple_of,
                                      dropout=config.dropout, bias=config.bias)
        self.norm1 = nn.LayerNorm(config.hidden_size)
        self.norm2 = nn.LayerNorm(config.hidden_size)

    def forward(self, x, mask=None):
        x = x + self.attn(self.norm1(x), mask)
        return x + self.ff(self.norm2(x))


class GPT(nn.Module):
    def __init__(self, config: Config) -> None:
        super().__init__()
        if config.hidden_size % config.num_attention_heads != 0:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        if config.mlp not in MLP_MAP:
            raise ValueError(f"mlp must be one of {sorted(MLP_MAP)}, got {config.mlp!r}")
        self.config = config
        self.word_emb = nn.Embedding(config.vocab_size, config.hidden_size)
        self.pos_emb = nn.Embedding(config.max_sequence_length, config.hidden_size)
        self.layers = nn.ModuleList([Block(config) for _ in range(config.num_hidden_layers)])
        self.norm = nn.LayerNorm(config.hidden_size)
        self.vocab_proj = Linear(config.hidden_size, config.vocab_size, bias=False)
        self.mask = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        seq = check_token_ids(x, self.config.max_sequence_length)
        h = self.word_emb(x) + self.pos_emb(torch.arange(seq, device=x.device))
        for layer in self.layers:
            h = layer(h, self.mask)
        return self.vocab_proj(self.norm(h))
