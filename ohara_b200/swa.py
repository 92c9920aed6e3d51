"""Sliding-window (local causal) attention helpers (reference: ohara/swa.py:7-79)."""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor


def make_swa_mask(seq_len: int, window_size: int, *, device: torch.device,
                  dtype: torch.dtype) -> Tensor:
    """Additive ``(T, T)`` mask: 0 where ``0 <= i - j < window_size``, ``-inf`` elsewhere."""
    offset = torch.arange(seq_len, device=device)[:, None] - torch.arange(seq_len, device=device)
    allowed = (offset >= 0) & (offset < window_size)
    return torch.full((seq_len, seq_len), float("-inf"), device=device, dtype=dtype).masked_fill(
        allowed, 0.0)


def sliding_window_attention_with_mask(q: Tensor, k: Tensor, v: Tensor, window_size: int = 16):
    """Unscaled masked attention over ``(B, T, D)`` tensors (explicit ``T x T`` scores)."""
    mask = make_swa_mask(q.shape[1], window_size, device=q.device, dtype=q.dtype)
    return F.softmax(q @ k.transpose(-1, -2) + mask, dim=-1) @ v


def sliding_window_flex_attention(q: Tensor, k: Tensor, v: Tensor, window_size: int = 16, *,
                                  block_size: int = 128, enable_gqa: bool = False):
    """Same computation through ``torch.nn.attention.flex_attention`` with a block mask (skips
    fully-masked blocks). Accepts ``(B, T, D)`` or ``(B, H, T, D)``."""
    from torch.nn.attention import flex_attention as flex

    def inside(batch, head, q_idx, kv_idx):
        return (kv_idx <= q_idx) & ((q_idx - kv_idx) < window_size)

    headless = q.dim() == 3
    if headless:
        q, k, v = q.unsqueeze(1), k.unsqueeze(1), v.unsqueeze(1)
    block_mask = flex.create_block_mask(mask_mod=inside, B=q.shape[0], H=q.shape[1],
                                        Q_LEN=q.shape[2], KV_LEN=k.shape[2], device=q.device,
                                        BLOCK_SIZE=block_size)
    out = flex.flex_attention(q, k, v, block_mask=block_mask, enable_gqa=enable_gqa)
    return out.squeeze(1) if headless else out


def compare_swa_mask_vs_flex(q: Tensor, k: Tensor, v: Tensor, *, window_size: int,
                             block_size: int = 128):
    """Both implementations and their largest absolute difference."""
    dense = sliding_window_attention_with_mask(q, k, v, window_size=window_size)
    blocked = sliding_window_flex_attention(q, k, v, window_size=window_size, block_size=block_size)
    return dense, blocked, (dense - blocked).abs().max().item()
