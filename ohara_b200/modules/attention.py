"""Standalone causal multi-head self-attention block with biases and optional RoPE
(reference: ohara/modules/attention.py:22-135). ``verbose=True`` also returns the attention
matrix, which forces the explicit softmax path."""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200 import ops
from ohara_b200.embeddings_pos.rotary import apply_rope
from ohara_b200.modules.mlp import Linear


class CausalAttention(nn.Module):
    def __init__(self, d_model: int, num_heads: int, attn_dropout: float = 0.0,
                 res_dropout: float = 0.0, idx: int | None = None) -> None:
        super().__init__()
        if d_model % num_heads != 0:
            raise ValueError("d_model must be divisible by num_heads")
        self.num_heads = num_heads
        self.head_dim = d_model // num_heads
        self.idx = idx
        self.key = Linear(d_model, d_model)
        self.query = Linear(d_model, d_model)
        self.value = Linear(d_model, d_model)
        self.proj = Linear(d_model, d_model)
        self.attn_dropout = nn.Dropout(attn_dropout)
        self.res_dropout = nn.Dropout(res_dropout)
        self.reset_parameters()

    def forward(self, x: Tensor, mask: Tensor | None = None, freqs_cis=None, verbose: bool = False,
                **kwargs):
        batch, seq_len, d_model = x.shape
        shape = (batch, seq_len, self.num_heads, self.head_dim)
        q, k, v = self.query(x).view(shape), self.key(x).view(shape), self.value(x).view(shape)
        if freqs_cis is not None:
            q, k = apply_rope(q, k, freqs_cis)
        weights = None
        if verbose or mask is not None:
            qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
            scores = torch.matmul(qh, kh.transpose(2, 3)) / math.sqrt(self.head_dim)
            if mask is not None:
                scores = scores + mask[:, :, :seq_len, :seq_len]
            else:
                keep = torch.ones(seq_len, seq_len, dtype=torch.bool, device=x.device).tril()
                scores = scores.masked_fill(~keep, float("-inf"))
            weights = F.softmax(scores.float(), dim=-1).type_as(kh)
            out = torch.matmul(self.attn_dropout(weights), vh).transpose(1, 2)
        else:
            out = ops.attention(q, k, v, causal=True, dropout_p=self.attn_dropout.p,
                                training=self.training)
        out = self.res_dropout(self.proj(out.reshape(batch, seq_len, d_model)))
        if verbose:
            return out, {"idx": self.idx, "attn_mtx": weights}
        return out

    def reset_parameters(self, init_std: float | None = None, factor: float = 1.0) -> None:
        std = init_std or self.head_dim**-0.5
        for layer in (self.key, self.query, self.value):
            nn.init.trunc_normal_(layer.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
        nn.init.trunc_normal_(self.proj.weight, mean=0.0, std=std / factor, a=-3 * std, b=3 * std)


CasualAttention = CausalAttention  # historic spelling kept as an alias
Attention = CausalAttention
