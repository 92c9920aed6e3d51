"""Gemma-style decoder: fused biased ``qkv_proj``, multi-/grouped-query attention, GEGLU
feed-forward, RMSNorm blocks with a LayerNorm at the end, tied embeddings
(reference: ohara/models/gemma.py:15-184)."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200 import ops
from ohara_b200.embeddings_pos.rotary import apply_rope, precompute_freqs_cis
from ohara_b200.modules.mlp import GEGLU, Linear
from ohara_b200.modules.norm import RMSNorm

from ._blocks import check_token_ids


@dataclass
class GemmaConfig:
    vocab_size: int = 51200
    max_sequence_length: int = 2048
    hidden_size: int = 2048
    intermediate_size = 16 * 2048  # class attribute, not a dataclass field (as in the reference)
    num_attention_heads: int = 32
    num_key_value_heads: int = 1
    num_hidden_layers: int = 32
    dropout: float = 0.2
    multiple_of: int = 4
    bias: bool = True
    eps: float = 1e-5
    rotary_dim: float = 0.4


class GemmaAttention(nn.Module):
    def __init__(self, hidden_size: int, num_attention_heads: int, num_key_value_heads: int):
        super().__init__()
        assert num_attention_heads % num_key_value_heads == 0
        self.num_attention_heads = num_attention_heads
        self.num_key_value_heads = num_key_value_heads
        self.num_queries_per_kv = num_attention_heads // num_key_value_heads
        self.hidden_size = hidden_size
        self.head_dim = hidden_size // num_attention_heads
        self.q_size = num_attention_heads * self.head_dim
        self.kv_size = num_key_value_heads * self.head_dim
        self.scaling = self.head_dim**-0.5
        self.qkv_proj = Linear(hidden_size, self.q_size + 2 * self.kv_size)
        self.o_proj = Linear(self.q_size, hidden_size)

    def forward(self, x: Tensor, freqs_cis, mask: Tensor | None = None) -> Tensor:
        batch, seq, _ = x.shape
        q, k, v = self.qkv_proj(x).split([self.q_size, self.kv_size, self.kv_size], dim=-1)
        q = q.reshape(batch, seq, self.num_attention_heads, self.head_dim)
        k = k.reshape(batch, seq, self.num_key_value_heads, self.head_dim)
        v = v.reshape(batch, seq, self.num_key_value_heads, self.head_dim)
        q, k = apply_rope(q, k, freqs_cis)
        out = ops.attention(q, k, v.to(q.dtype), causal=True, scale=self.scaling)
        return self.o_proj(out.reshape(batch, seq, self.q_size))


class Block(nn.Module):
    def __init__(self, config: GemmaConfig):
        super().__init__()
        self.self_attn = GemmaAttention(config.hidden_size, config.num_attention_heads,
                                        config.num_key_value_heads)
        self.mlp = GEGLU(dim=config.hidden_size, hidden_dim=config.intermediate_size)
        self.ln1 = RMSNorm(config.hidden_size, eps=config.eps)
        self.ln2 = RMSNorm(config.hidden_size, eps=config.eps)

    def forward(self, x: Tensor, freqs_cis, mask: Tensor | None) -> Tensor:
        x = x + self.self_attn(self.ln1(x), freqs_cis=freqs_cis, mask=mask)
        return x + self.mlp(self.ln2(x))


class Gemma(nn.Module):
    def __init__(self, config: GemmaConfig) -> None:
        super().__init__()
        if config.hidden_size % config.num_attention_heads != 0:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        self.config = config
        self.token_emb = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([Block(config) for _ in range(config.num_hidden_layers)])
        self.norm = nn.LayerNorm(config.hidden_size)
        self.vocab_proj = Linear(config.hidden_size, config.vocab_size, bias=False)
        self.token_emb.weight = self.vocab_proj.weight
        cos, sin = precompute_freqs_cis(config.hidden_size // config.num_attention_heads,
                                        config.max_sequence_length * 2)
        self.register_buffer("freq_cos", cos, persistent=False)
        self.register_buffer("freq_sin", sin, persistent=False)
        self.mask = None  # causal masking happens inside the attention op

    def forward(self, x: Tensor) -> Tensor:
        seq = check_token_ids(x, self.config.max_sequence_length)
        freqs = (self.freq_cos[:seq], self.freq_sin[:seq])
        h = self.token_emb(x)
        for layer in self.layers:
            h = layer(h, freqs, self.mask)
        return self.vocab_proj(self.norm(h))
