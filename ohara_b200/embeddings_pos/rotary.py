"""Rotary position embeddings.

Two entry points, matching the reference surface (ohara/embeddings_pos/rotary.py:24-184):

* ``precompute_freqs_cis`` + ``apply_rope``: table-driven, *interleaved pair* rotation
  ``(x0, x1), (x2, x3), ...`` on ``(batch, seq, heads, head_dim)`` tensors. On a CUDA device the
  rotation of q and k runs as one sm_100a kernel (forward and backward); on CPU it is the fp32
  reference that the kernel is tested against.
* ``RoPE``: module that builds its own angles, supports partial rotation and a position offset.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
from torch import Tensor


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0) -> tuple[Tensor, Tensor]:
    """Return ``(cos, sin)`` tables of shape ``(end, dim // 2)`` in fp32."""
    half = dim // 2
    exponents = torch.arange(0, dim, 2)[:half].float() / dim
    inv_freq = 1.0 / (theta**exponents)
    angles = torch.outer(torch.arange(end, dtype=torch.float32), inv_freq)
    return torch.cos(angles), torch.sin(angles)


def rope_reference(x: Tensor, cos: Tensor, sin: Tensor, inverse: bool = False) -> Tensor:
    """fp32 interleaved-pair rotation of one tensor ``(B, T, H, D)``; ``inverse`` rotates by −θ."""
    seq_len = x.shape[1]
    cos = cos[:seq_len].view(1, seq_len, 1, -1)
    sin = sin[:seq_len].view(1, seq_len, 1, -1)
    if inverse:
        sin = -sin
    pairs = x.float().reshape(*x.shape[:-1], -1, 2)
    even, odd = pairs[..., 0], pairs[..., 1]
    rotated = torch.stack((even * cos - odd * sin, even * sin + odd * cos), dim=-1)
    return rotated.flatten(-2).to(x.dtype)


def reshape_for_broadcast(freqs_cis: Tensor, x: Tensor) -> Tensor:
    """View a ``(seq_len, width)`` table so that it broadcasts against ``x (batch, seq_len, ...,
    width)``: the sequence and the last dimension are kept, every other one becomes 1 (helper of
    the reference's public surface: ohara/embeddings_pos/rotary.py:41-52)."""
    if x.dim() < 2 or tuple(freqs_cis.shape) != (x.shape[1], x.shape[-1]):
        raise ValueError(f"table of shape {tuple(freqs_cis.shape)} does not match input "
                         f"{tuple(x.shape)} (expected {(x.shape[1], x.shape[-1])})")
    last = x.dim() - 1
    return freqs_cis.view([size if axis in (1, last) else 1 for axis, size in enumerate(x.shape)])


def apply_rope(q: Tensor, k: Tensor, cis: tuple[Tensor, Tensor]) -> tuple[Tensor, Tensor]:
    """Rotate ``q`` and ``k`` (``(B, T, H, D)``) by tables already sliced to their positions."""
    cos, sin = cis
    seq_len = q.shape[1]
    if cos.shape[0] < seq_len or cos.shape[-1] * 2 != q.shape[-1]:
        raise ValueError(
            f"rotary table {tuple(cos.shape)} does not cover q of shape {tuple(q.shape)}"
        )
    if q.is_cuda:
        from ohara_b200.ops import rope_qk

        return rope_qk(q, k, cos, sin)
    return rope_reference(q, cos, sin), rope_reference(k, cos, sin).to(q.dtype)


class RoPE(nn.Module):
    """Self-contained rotary module (reference: ohara/embeddings_pos/rotary.py:96-184).

    ``traditional=False`` pairs feature ``i`` with ``i + dims/2``; ``traditional=True`` pairs
    neighbours. Only the first ``dims`` features rotate; the rest pass through.
    """

    def __init__(
        self, dims: int, traditional: bool = False, base: float = 10000, scale: float = 1.0
    ) -> None:
        super().__init__()
        if dims < 2 or dims % 2:
            raise ValueError(f"RoPE dims must be a positive even number, got {dims}")
        self.dims = dims
        self.traditional = traditional
        self.base = base
        self.scale = scale

    def extra_repr(self) -> str:
        return f"{self.dims}, traditional={self.traditional}"

    @staticmethod
    def create_cos_sin_theta(
        num_positions: int,
        dims: int,
        offset: int = 0,
        base: float = 10000,
        scale: float = 1.0,
        dtype: torch.dtype = torch.float32,
        device: torch.device | str | None = None,
    ) -> tuple[Tensor, Tensor]:
        half = dims // 2
        pos = torch.arange(offset, num_positions, dtype=dtype, device=device) * scale
        freqs = torch.exp(
            -torch.arange(0.0, half, dtype=dtype, device=device) * (math.log(base) / half)
        )
        theta = pos[:, None] * freqs[None, :]
        return torch.cos(theta), torch.sin(theta)

    def forward(self, x: Tensor, offset: int = 0) -> Tensor:
        shape = x.shape
        x = x.reshape(-1, shape[-2], shape[-1])
        cos, sin = self.create_cos_sin_theta(
            x.shape[1] + offset,
            self.dims,
            offset=offset,
            base=self.base,
            scale=self.scale,
            dtype=x.dtype,
            device=x.device,
        )
        if self.traditional:
            if self.dims < x.shape[-1]:
                raise NotImplementedError("RoPE doesn't implement partial traditional application")
            a, b = x[..., ::2], x[..., 1::2]
            out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)
        else:
            half = self.dims // 2
            a, b = x[..., :half], x[..., half : self.dims]
            parts = [a * cos - b * sin, a * sin + b * cos]
            if self.dims < x.shape[-1]:
                parts.append(x[..., self.dims :])
            out = torch.cat(parts, dim=-1)
        return out.reshape(shape)
