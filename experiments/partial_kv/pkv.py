"""Attention variants that shrink the key/value cache by *sharing numbers between keys and values*
(reference: experiments/partial_kv/pkv.py:48-205).

* :class:`KeyValueTiedAttention`: one projection serves as both key and value (after the rotary
  rotation of the key), so a token caches ``head_dim`` numbers per head instead of ``2 * head_dim``.
* :class:`PartialKVAttention`: a token caches three half-width pieces per head, ``shared``,
  ``key`` and ``value``; the key the scores use is ``[shared | rope(key)]`` and the value they
  weight is ``[shared | value]`` (``1.5 * head_dim`` numbers instead of ``2 * head_dim``). Only the
  second half of a query is rotated, matching the rotated half of the key.

Both take ``(x, freqs)`` with the rotary tables of the *rotated width* and are causal. A plain
multi-head :class:`FullAttention` with the same interface serves as the baseline, and
:func:`cache_floats_per_token` gives the cache sizes that motivate the variants.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200.embeddings_pos.rotary import apply_rope


def _heads(x: Tensor, heads: int) -> Tensor:
    batch, steps, width = x.shape
    return x.view(batch, steps, heads, width // heads)


def _attend(q: Tensor, k: Tensor, v: Tensor, dropout: float, training: bool) -> Tensor:
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                         dropout_p=dropout if training else 0.0, is_causal=True)
    return out.transpose(1, 2).flatten(2)


class FullAttention(nn.Module):
    cache_factor = 2.0

    def __init__(self, d_model: int, num_heads: int, dropout: float = 0.0, bias: bool = False):
        super().__init__()
        self.num_heads, self.dropout = num_heads, dropout
        self.query = nn.Linear(d_model, d_model, bias)
        self.key = nn.Linear(d_model, d_model, bias)
        self.value = nn.Linear(d_model, d_model, bias)
        self.proj = nn.Linear(d_model, d_model, bias)

    def forward(self, x: Tensor, freqs: tuple[Tensor, Tensor]) -> Tensor:
        q, k = apply_rope(_heads(self.query(x), self.num_heads), _heads(self.key(x), self.num_heads),
                          freqs)
        return self.proj(_attend(q, k, _heads(self.value(x), self.num_heads), self.dropout,
                                 self.training))


class KeyValueTiedAttention(nn.Module):
    """Values are the (rotated) keys."""

    cache_factor = 1.0

    def __init__(self, d_model: int, num_heads: int, dropout: float = 0.0, bias: bool = False):
        super().__init__()
        self.num_heads, self.dropout = num_heads, dropout
        self.query = nn.Linear(d_model, d_model, bias)
        self.key = nn.Linear(d_model, d_model, bias)
        self.proj = nn.Linear(d_model, d_model, bias)

    def forward(self, x: Tensor, freqs: tuple[Tensor, Tensor]) -> Tensor:
        q, k = apply_rope(_heads(self.query(x), self.num_heads), _heads(self.key(x), self.num_heads),
                          freqs)
        return self.proj(_attend(q, k, k, self.dropout, self.training))


class PartialKVAttention(nn.Module):
    """Keys and values share half of their width. ``freqs`` are rotary tables for ``head_dim / 2``."""

    cache_factor = 1.5

    def __init__(self, d_model: int, num_heads: int, dropout: float = 0.0, bias: bool = False):
        super().__init__()
        head_dim = d_model // num_heads
        if d_model % num_heads or head_dim % 4:
            raise ValueError("head_dim must be a multiple of 4 (two halves, each rotated in pairs)")
        self.num_heads, self.dropout, self.half = num_heads, dropout, head_dim // 2
        self.query = nn.Linear(d_model, d_model, bias)
        self.keyvalue = nn.Linear(d_model, 3 * num_heads * self.half, bias)  # key | shared | value
        self.proj = nn.Linear(d_model, d_model, bias)

    def cached(self, x: Tensor, freqs: tuple[Tensor, Tensor]) -> tuple[Tensor, Tensor, Tensor]:
        """The three pieces a decoder would cache per token and head: rotated key half, shared
        half, value half, each ``(batch, steps, heads, head_dim / 2)``."""
        key, shared, value = (_heads(t, self.num_heads) for t in self.keyvalue(x).chunk(3, dim=-1))
        _, key = apply_rope(key, key, freqs)
        return key, shared, value

    def forward(self, x: Tensor, freqs: tuple[Tensor, Tensor]) -> Tensor:
        plain, rotated = (_heads(t, self.num_heads) for t in self.query(x).chunk(2, dim=-1))
        rotated, _ = apply_rope(rotated, rotated, freqs)
        key, shared, value = self.cached(x, freqs)
        q = torch.cat([plain, rotated], dim=-1)
        k = torch.cat([shared, key], dim=-1)
        v = torch.cat([shared, value], dim=-1)
        return self.proj(_attend(q, k, v, self.dropout, self.training))


ATTENTION = {"attention": FullAttention, "kattention": KeyValueTiedAttention,
             "partial_kv": PartialKVAttention}


def cache_floats_per_token(kind: str, d_model: int, num_layers: int) -> int:
    """Numbers a decoder keeps per token for ``num_layers`` layers of attention ``kind``."""
    return int(ATTENTION[kind].cache_factor * d_model) * num_layers
