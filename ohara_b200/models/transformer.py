"""Configurable llama-style transformer plus ``ModelingLM``, a Hub-serialisable wrapper
(``save_pretrained`` / ``push_to_hub`` / ``from_pretrained`` through
``huggingface_hub.PyTorchModelHubMixin``). Reference: ohara/models/transformer.py:24-211."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
from huggingface_hub import PyTorchModelHubMixin

from ohara_b200.embeddings_pos.rotary import precompute_freqs_cis
from ohara_b200.modules.mlp import GLU, MLP, Linear
from ohara_b200.modules.norm import RMSNorm

from ._blocks import SelfAttention, init_normal


@dataclass
class Config:
    vocab_size: int
    seq_len: int
    d_model: int
    hidden_dim: int
    num_heads: int
    num_kv_heads: int = 0
    num_layers: int = 4
    dropout: float = 0.2
    bias: bool = False
    weight_tying: bool = False
    activation: str = "silu"
    mlp: str = "GLU"  # "MLP" or "GLU"


MLP_BLOCK = {"MLP": MLP, "GLU": GLU}


class Attention(SelfAttention):
    def __init__(self, config: Config):
        super().__init__(config.d_model, config.num_heads, kv_heads=config.num_kv_heads,
                         bias=config.bias, dropout=config.dropout)

    def forward(self, x, mask, freqs_cis):
        return super().forward(x, freqs_cis)


class Block(nn.Module):
    def __init__(self, config: Config):
        super().__init__()
        self.attn = Attention(config)
        self.ff = MLP_BLOCK[config.mlp](dim=config.d_model, hidden_dim=config.hidden_dim,
                                        dropout=config.dropout, bias=config.bias,
                                        activation_fn=config.activation)
        self.norm1 = RMSNorm(config.d_model)
        self.norm2 = RMSNorm(config.d_model)

    def forward(self, x, mask, freqs_cis):
        x = x + self.attn(self.norm1(x), mask, freqs_cis)
        return x + self.ff(self.norm2(x))


class Transformer(nn.Module):
    def __init__(self, config: Config, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.config = config
        self.token_emb = nn.Embedding(config.vocab_size, config.d_model)
        self.layers = nn.ModuleList([Block(config) for _ in range(config.num_layers)])
        self.norm = RMSNorm(config.d_model)
        self.vocab_proj = Linear(config.d_model, config.vocab_size, bias=False)
        if config.weight_tying:
            self.token_emb.weight = self.vocab_proj.weight
        cos, sin = precompute_freqs_cis(config.d_model // config.num_heads, config.seq_len * 2)
        self.register_buffer("freq_cos", cos)
        self.register_buffer("freq_sin", sin)
        self.mask = None
        self.apply(init_normal)

    def forward(self, x: torch.Tensor):
        seq = x.shape[1]
        freqs = (self.freq_cos[:seq], self.freq_sin[:seq])
        h = self.token_emb(x)
        for layer in self.layers:
            h = layer(h, self.mask, freqs)
        return self.vocab_proj(self.norm(h))


class ModelingLM(nn.Module, PyTorchModelHubMixin):
    def __init__(self, config: Config | dict) -> None:
        super().__init__()
        if isinstance(config, dict):
            config = Config(**config)
        self.config = config
        self.model = Transformer(config)

    def forward(self, x: torch.Tensor):
        return self.model(x)
