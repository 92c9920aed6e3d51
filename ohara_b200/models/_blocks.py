"""Attention block shared by the small model zoo (GPT, RoFormer, Transformer).

Separate ``key / query / value / proj`` linears (the parameter names every zoo checkpoint uses),
optional rotary embedding and grouped-query heads, computed in the ``(B, T, H, D)`` layout through
:func:`ohara_b200.ops.attention` — so on CUDA bf16 the flash-attention kernels run, with no head
transposes, KV expansion or mask tensors.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200 import ops
from ohara_b200.embeddings_pos.rotary import apply_rope
from ohara_b200.modules.mlp import Linear


class SelfAttention(nn.Module):
    def __init__(self, width: int, heads: int, kv_heads: int = 0, bias: bool = False,
                 dropout: float = 0.0) -> None:
        super().__init__()
        self.num_heads = heads
        self.head_dim = width // heads
        self.num_kv_heads = kv_heads or heads
        if heads % self.num_kv_heads:
            raise ValueError("num_kv_heads must divide num_heads")
        self.key = Linear(width, self.head_dim * self.num_kv_heads, bias=bias)
        self.query = Linear(width, self.head_dim * heads, bias=bias)
        self.value = Linear(width, self.head_dim * self.num_kv_heads, bias=bias)
        self.proj = Linear(width, width, bias=bias)
        self.attn_dropout = nn.Dropout(dropout)
        self.res_dropout = nn.Dropout(dropout)

    def forward(self, x: Tensor, freqs_cis=None) -> Tensor:
        batch, seq, width = x.shape
        q = self.query(x).view(batch, seq, self.num_heads, self.head_dim)
        k = self.key(x).view(batch, seq, self.num_kv_heads, self.head_dim)
        v = self.value(x).view(batch, seq, self.num_kv_heads, self.head_dim)
        if freqs_cis is not None:
            q, k = apply_rope(q, k, freqs_cis)
        out = ops.attention(q, k, v.to(q.dtype), causal=True, dropout_p=self.attn_dropout.p,
                            training=self.training)
        return self.res_dropout(self.proj(out.reshape(batch, seq, width)))


def check_token_ids(x: Tensor, limit: int) -> int:
    if x.ndim != 2:
        raise ValueError("input token IDs must have shape (batch, sequence)")
    if x.size(1) > limit:
        raise ValueError("input exceeds max_sequence_length")
    return x.size(1)


def init_normal(module: nn.Module, std: float = 0.02) -> None:
    if isinstance(module, nn.Linear):
        nn.init.normal_(module.weight, mean=0.0, std=std)
        if module.bias is not None:
            nn.init.zeros_(module.bias)
    elif isinstance(module, nn.Embedding):
        nn.init.normal_(module.weight, mean=0.0, std=std)
