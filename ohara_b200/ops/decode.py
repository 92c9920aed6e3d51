"""Serving ops on the kernels of ``csrc/decode.cu``: fused RoPE + KV-cache append, split-KV decode
attention over the cache in place, and the fused temperature / top-k / top-p sampler.

``position`` arguments are either a Python int (eager decoding) or a one-element int32 CUDA tensor
(the kernels read the value on the device, so the step can be replayed from a CUDA graph).
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

from ._ext import ext


def fused_decode_supported(q: Tensor, cache) -> bool:
    """True when the serving kernels can run this layer's decode step."""
    if not (q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 4):
        return False
    heads, dim = q.shape[2], q.shape[3]
    kv_heads = cache.key.shape[2]
    store_ok = cache.key.dtype in (torch.bfloat16, torch.int8) and cache.key.is_cuda
    return store_ok and dim in (64, 128) and heads % kv_heads == 0 and heads // kv_heads in (1, 2, 4, 8)


def _split_position(position):
    if isinstance(position, Tensor):
        return 0, position
    return int(position), None


def _stats(cache) -> list[Tensor]:
    if not cache.int8:
        return []
    return [cache.key_scale, cache.key_min, cache.value_scale, cache.value_min]


def rope_append(q: Tensor, k: Tensor, v: Tensor, cache, cos: Tensor, sin: Tensor, position) -> Tensor:
    """Rotate ``q``/``k`` (``(B, T, H, D)``) at absolute positions ``position + t`` using the *full*
    fp32 tables ``cos``/``sin``, write rotated ``k`` and ``v`` into ``cache`` at those positions
    (quantising when the cache is int8) and return the rotated ``q``."""
    pos, pos_dev = _split_position(position)
    return ext().rope_append(q.contiguous(), k.contiguous(), v.contiguous(), cache.key, cache.value,
                             _stats(cache), cos, sin, pos, pos_dev)


def decode_attention(q: Tensor, cache, position, scale: float | None = None) -> Tensor:
    """Attention of one query token per sequence, ``q (B, 1, H, D)``, over cache positions
    ``0 .. position`` inclusive. Returns ``(B, 1, H, D)``."""
    batch, one, heads, dim = q.shape
    pos, pos_dev = _split_position(position)
    scale = scale if scale is not None else 1.0 / math.sqrt(dim)
    out = ext().decode_attention(q.reshape(batch, heads, dim), cache.key, cache.value, _stats(cache),
                                 pos + 1, pos_dev, float(scale), 0)
    return out.view(batch, one, heads, dim)


def sample(logits: Tensor, *, temperature: float, top_k: int = 0, top_p: float = 1.0,
           valid_vocab: int | None = None, uniforms: Tensor | None = None,
           out: Tensor | None = None, next_input: Tensor | None = None,
           counters: Tensor | None = None) -> Tensor:
    """Sample one token per row of ``logits (rows, vocab)``.

    ``uniforms`` holds one U[0,1) number per row (``(steps, rows)`` when ``counters`` selects the
    step on the device); ``None`` or ``temperature == 0`` means greedy. Token ids at or above
    ``valid_vocab`` are never produced. Returns ``out`` (``(rows, steps)`` int64; a fresh
    ``(rows, 1)`` tensor when not given). With ``counters`` (int32 ``[step, position, done]`` on the
    device) the kernel writes column ``step``, copies the token to ``next_input`` and advances
    ``step`` and ``position`` itself.
    """
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, 1, device=logits.device, dtype=torch.int64)
    if temperature > 0 and uniforms is None:
        uniforms = torch.rand(rows, device=logits.device, dtype=torch.float32)
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    ext().sample_tokens(logits, vocab if valid_vocab is None else valid_vocab, float(temperature),
                        int(top_k), float(top_p), uniforms if temperature > 0 else None, out,
                        next_input, counters, None)
    return out
