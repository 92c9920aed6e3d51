"""Scaled dot-product attention with native grouped-query heads.

Layout is ``(batch, seq, heads, head_dim)`` throughout — the layout the QKV projections produce —
so no transposes or KV head expansion are materialised. ``causal=True`` aligns the mask to the
*end* of the key sequence (query ``i`` of ``T`` sees keys ``<= S - T + i``), which is plain causal
attention when ``S == T`` and the KV-cache rule ``key_pos <= query_pos`` when ``S > T``.

CUDA bf16 inputs run the flash-attention kernels (forward and backward); everything else runs the
fp32 reference below, which is also the kernels' test oracle (reference slow path:
ohara/models/llama.py:124-135).
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

from ._ext import ext


def attention_reference(q: Tensor, k: Tensor, v: Tensor, causal: bool = True,
                        scale: float | None = None, dropout_p: float = 0.0,
                        training: bool = False) -> Tensor:
    """fp32 softmax(QK^T * scale + mask) V with grouped-query expansion. Shapes as in `attention`."""
    b, t, h, d = q.shape
    s, hk = k.shape[1], k.shape[2]
    group = h // hk
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qf = q.float().permute(0, 2, 1, 3)  # (b, h, t, d)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qpos = torch.arange(t, device=q.device) + (s - t)
        kpos = torch.arange(s, device=q.device)
        scores = scores.masked_fill(~(kpos[None, :] <= qpos[:, None]), float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    if dropout_p > 0.0 and training:
        probs = torch.nn.functional.dropout(probs, dropout_p)
    out = torch.matmul(probs, vf)
    return out.permute(0, 2, 1, 3).to(q.dtype)


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, causal: bool, scale: float):
        out, lse = ext().flash_attn_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal = causal
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = ext().flash_attn_bwd(dout.contiguous(), q, k, v, out, lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


class _RopeAttentionFn(torch.autograd.Function):
    """Rotary embedding of q and k plus causal attention on a fused ``q | k | v`` projection
    ``(B, T, (H + 2 Hk) D)``. q, k and v are read as column slices of it (no copies); the backward
    pass returns one gradient for the whole projection: the value gradient is stored into its
    columns by the attention kernel, the un-rotated query / key gradients by the rotary kernel."""

    @staticmethod
    def forward(ctx, qkv: Tensor, cos: Tensor, sin: Tensor, heads: int, kv_heads: int, dim: int,
                causal: bool, scale: float):
        C = ext()
        batch, seq, _ = qkv.shape
        nq, nk = heads * dim, kv_heads * dim
        q = qkv[..., :nq].view(batch, seq, heads, dim)
        k = qkv[..., nq:nq + nk].view(batch, seq, kv_heads, dim)
        v = qkv[..., nq + nk:].view(batch, seq, kv_heads, dim)
        q_rot, k_rot = C.rope(q, k, cos, sin, False)
        out, lse = C.flash_attn_fwd(q_rot, k_rot, v, causal, scale)
        ctx.save_for_backward(q_rot, k_rot, qkv, out, lse, cos, sin)
        ctx.meta = (heads, kv_heads, dim, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        C = ext()
        q_rot, k_rot, qkv, out, lse, cos, sin = ctx.saved_tensors
        heads, kv_heads, dim, causal, scale = ctx.meta
        batch, seq, _ = qkv.shape
        nq, nk = heads * dim, kv_heads * dim
        v = qkv[..., nq + nk:].view(batch, seq, kv_heads, dim)
        dqkv = torch.empty_like(qkv)
        dv = dqkv[..., nq + nk:].view(batch, seq, kv_heads, dim)
        dk_rot = torch.empty_like(k_rot)
        dq_rot, _, _ = C.flash_attn_bwd(dout.contiguous(), q_rot, k_rot, v, out, lse, causal, scale,
                                        dk_rot, dv)
        C.rope(dq_rot, dk_rot, cos, sin, True,
               dqkv[..., :nq].view(batch, seq, heads, dim),
               dqkv[..., nq:nq + nk].view(batch, seq, kv_heads, dim))
        return dqkv, None, None, None, None, None, None, None


def rope_attention(qkv: Tensor, cos: Tensor, sin: Tensor, heads: int, kv_heads: int, dim: int,
                   causal: bool = True, scale: float | None = None) -> Tensor:
    """Rotate and attend on a fused ``q | k | v`` projection ``(B, T, (heads + 2 kv_heads) dim)``
    with rotary tables already sliced to the tokens' positions; returns ``(B, T, heads, dim)``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(dim)
    batch, seq, width = qkv.shape
    if width != (heads + 2 * kv_heads) * dim:
        raise ValueError("fused projection width does not match the head counts")
    if (qkv.is_cuda and qkv.dtype == torch.bfloat16 and dim in (64, 128) and qkv.is_contiguous()
            and width % 8 == 0):
        cos = cos[:seq].float().contiguous()
        sin = sin[:seq].float().contiguous()
        return _RopeAttentionFn.apply(qkv, cos, sin, heads, kv_heads, dim, causal, float(scale))
    from ohara_b200.embeddings_pos.rotary import apply_rope

    nq, nk = heads * dim, kv_heads * dim
    q = qkv[..., :nq].reshape(batch, seq, heads, dim)
    k = qkv[..., nq:nq + nk].reshape(batch, seq, kv_heads, dim)
    v = qkv[..., nq + nk:].reshape(batch, seq, kv_heads, dim)
    q, k = apply_rope(q, k, (cos, sin))
    return attention(q, k.to(q.dtype), v.to(q.dtype), causal=causal, scale=scale)


def _kernel_ok(q: Tensor, k: Tensor, v: Tensor) -> bool:
    d = q.shape[-1]
    return (
        q.is_cuda
        and q.dtype == k.dtype == v.dtype == torch.bfloat16
        and d in (64, 128)
        and q.shape[2] % k.shape[2] == 0
    )


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, scale: float | None = None,
              dropout_p: float = 0.0, training: bool = False) -> Tensor:
    """``q (B,T,H,D)``, ``k/v (B,S,Hk,D)`` → ``(B,T,H,D)``."""
    if q.dim() != 4 or k.dim() != 4 or v.shape != k.shape:
        raise ValueError("attention expects (batch, seq, heads, head_dim) tensors")
    if q.shape[2] % k.shape[2] != 0:
        raise ValueError("number of query heads must be a multiple of the number of KV heads")
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    use_dropout = dropout_p > 0.0 and training
    if _kernel_ok(q, k, v) and not use_dropout:
        return _FlashAttnFn.apply(q, k, v, causal, float(scale))
    if not q.is_cuda:
        # CPU tensors: PyTorch's fused attention, as the reference model uses
        # (ohara/models/llama.py:115-123). Its own causal mask is aligned to the first key, which
        # is the mask wanted here only when queries and keys cover the same positions; a single
        # query at the end of a cache sees every key, and any other offset gets an explicit mask.
        steps, keys = q.shape[1], k.shape[1]
        mask = None
        if causal and steps != keys and steps > 1:
            mask = (torch.arange(keys, device=q.device)[None, :]
                    <= torch.arange(keys - steps, keys, device=q.device)[:, None])
        group = q.shape[2] // k.shape[2]
        kt, vt = k.transpose(1, 2), v.transpose(1, 2)
        if group > 1:
            kt, vt = kt.repeat_interleave(group, dim=1), vt.repeat_interleave(group, dim=1)
        out = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), kt, vt, attn_mask=mask,
            dropout_p=dropout_p if use_dropout else 0.0,
            is_causal=causal and steps == keys, scale=scale)
        return out.transpose(1, 2)
    return attention_reference(q, k, v, causal, scale, dropout_p, training)
