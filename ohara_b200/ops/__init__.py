"""Functional ops backed by the hand-written sm_100a kernels.

Every op has two implementations selected by the *device of its inputs*: CUDA tensors run the
kernels from ``ohara_b200/csrc`` (tcgen05 GEMMs, fused norm/rope/activation/loss kernels); CPU
tensors run a plain fp32 PyTorch reference, which is also the oracle the kernels are tested against.
There is no third backend and no silent fallback: on a CUDA device a missing extension raises.

Mixed precision: parameters stay fp32 ("master" weights). Inside ``torch.autocast("cuda",
torch.bfloat16)`` — what ``OharaEngine.autocast_context()`` enters for ``bf16_mixed`` — the ops
compute in bf16 from a cached bf16 copy of each weight and keep activations in bf16.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

from ohara_b200.errors import CollectiveTimeout

from ._ext import ext

import os as _os

_FUSE_PROJECTIONS = _os.environ.get("OHARA_FUSED_PROJECTIONS", "1") != "0"

__all__ = [
    "add_rms_norm",
    "attention",
    "bf16_weight",
    "embedding",
    "fast_path",
    "linear",
    "linear_cross_entropy",
    "linear_cat",
    "linear_fanout",
    "rope_attention",
    "swiglu_cat",
    "matmul_nn",
    "matmul_nt",
    "matmul_tn",
    "rms_norm",
    "rope_qk",
    "swiglu",
    "check_status",
]


# --------------------------------------------------------------------------------------------------
# Precision helpers
# --------------------------------------------------------------------------------------------------
def fast_path(x: Tensor) -> bool:
    """True when ``x`` should run through the bf16 kernels: on CUDA and either already bf16 or
    inside a bf16 autocast region."""
    if not x.is_cuda:
        return False
    if x.dtype == torch.bfloat16:
        return True
    return torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16


def bf16_weight(weight: Tensor) -> Tensor:
    """bf16 compute copy of a parameter, cached on the parameter until it is modified in place.

    Optimizers in this package refresh the copy themselves while they update the fp32 master
    (``refresh_bf16_weight``); any other in-place change bumps the tensor version and the copy is
    rebuilt lazily with the cast kernel.
    """
    if weight.dtype == torch.bfloat16:
        return weight.detach()
    cached = getattr(weight, "_ohara_bf16", None)
    # ``param.data = tensor`` swaps the storage without bumping the version counter, so the key
    # carries the storage address as well.
    version = (weight._version, weight.data_ptr())
    if cached is not None and cached[0] == version and cached[1].device == weight.device:
        return cached[1]
    source = weight.detach()
    shadow = cached[1] if cached is not None and cached[1].shape == weight.shape else None
    if shadow is None or shadow.device != weight.device:
        shadow = torch.empty_like(source, dtype=torch.bfloat16)
    if source.dtype == torch.float32 and source.is_contiguous():
        ext().cast_bf16_into(source, shadow)
    else:
        shadow.copy_(source)
    weight._ohara_bf16 = (version, shadow)
    return shadow


def _f32_weight(weight: Tensor) -> Tensor:
    """Contiguous fp32 view of a norm weight; a low-precision parameter (a model converted to bf16
    for serving) gets a cached fp32 copy that is rebuilt only when the parameter changes."""
    source = weight.detach()
    if source.dtype == torch.float32:
        return source.contiguous()
    cached = getattr(weight, "_ohara_f32", None)
    version = (weight._version, weight.data_ptr())
    if cached is not None and cached[0] == version and cached[1].device == weight.device:
        return cached[1]
    copy = source.float().contiguous()
    weight._ohara_f32 = (version, copy)
    return copy


def refresh_bf16_weight(weight: Tensor, shadow: Tensor) -> None:
    """Record ``shadow`` as the up-to-date bf16 copy of ``weight`` (called by fused optimizers)."""
    weight._ohara_bf16 = ((weight._version, weight.data_ptr()), shadow)


def check_status(clear: bool = True) -> None:
    """Raise if any kernel recorded a timed-out wait since the last check (synchronises)."""
    code, block, count, _ = ext().status(clear)
    if code != 0:
        names = {
            1: "TMA data never arrived",
            2: "pipeline stage never released",
            3: "accumulator never completed",
            4: "accumulator never drained",
            5: "peer flag never written",
            6: "attention hand-off timed out",
            7: "bad kernel argument",
        }
        raise CollectiveTimeout(
            f"ohara_b200 kernel wait timed out: {names.get(code, code)} "
            f"(first in block {block}, {count} waits abandoned)"
        )


# --------------------------------------------------------------------------------------------------
# GEMM front-ends (bf16 in, bf16 or fp32 out)
# --------------------------------------------------------------------------------------------------
def _as_2d(x: Tensor) -> Tensor:
    return x.reshape(-1, x.shape[-1])


def _gemm_ready(t: Tensor) -> Tensor:
    """Return ``t`` with unit inner stride, 16-byte aligned base and row pitch."""
    if (
        t.stride(-1) != 1
        or (t.data_ptr() % 16)
        or any((t.stride(i) * t.element_size()) % 16 for i in range(t.dim() - 1))
    ):
        t = t.contiguous()
        if t.data_ptr() % 16:
            t = t.clone()
    return t


def matmul_nt(a: Tensor, b: Tensor, out: Tensor | None = None, out_dtype=torch.bfloat16,
              alpha: float = 1.0) -> Tensor:
    """``a (M,K) @ b (N,K)^T`` — the forward of a linear layer."""
    a, b = _gemm_ready(a), _gemm_ready(b)
    m, k = a.shape[-2:]
    n = b.shape[-2]
    if out is None:
        out = torch.empty((*a.shape[:-2], m, n), device=a.device, dtype=out_dtype)
    if (m <= 16 and a.dim() == 2 and b.dim() == 2 and alpha == 1.0
            and out.dtype == torch.bfloat16 and ext().gemv(a, b, out)):
        return out  # decode-sized input: the weight-streaming kernel beats the tensor-core set-up
    ext().gemm(a, b, out, m, n, k, False, False, 1, False, alpha, None, None)
    return out


def matmul_nn(a: Tensor, b: Tensor, out: Tensor | None = None, out_dtype=torch.bfloat16,
              alpha: float = 1.0) -> Tensor:
    """``a (M,K) @ b (K,N)`` — the input gradient of a linear layer (b = weight (out, in))."""
    a, b = _gemm_ready(a), _gemm_ready(b)
    m, k = a.shape[-2:]
    n = b.shape[-1]
    if out is None:
        out = torch.empty((*a.shape[:-2], m, n), device=a.device, dtype=out_dtype)
    ext().gemm(a, b, out, m, n, k, False, True, 1, False, alpha, None, None)
    return out


def _pick_splits(m: int, n: int, k: int) -> int:
    tiles = math.ceil(m / 128) * math.ceil(n / (256 if n > 128 else 128))
    if tiles >= 120:
        return 1
    k_blocks = math.ceil(k / 64)
    return max(1, min(148 // tiles, k_blocks // 8 if k_blocks >= 16 else 1, 32))


def matmul_tn(a: Tensor, b: Tensor, out: Tensor | None = None, accumulate: bool = False,
              alpha: float = 1.0) -> Tensor:
    """``a (K,M)^T @ b (K,N)`` in fp32 — the weight gradient of a linear layer (K = tokens).

    Split-K across the SMs with a TMA reduce-add epilogue; ``accumulate=True`` adds into ``out``.
    """
    a, b = _gemm_ready(a), _gemm_ready(b)
    k, m = a.shape[-2:]
    n = b.shape[-1]
    if out is None:
        out = torch.zeros((*a.shape[:-2], m, n), device=a.device, dtype=torch.float32)
        accumulate = True
    splits = _pick_splits(m, n, k) if a.dim() == 2 else 1
    if not accumulate:
        if splits == 1:
            ext().gemm(a, b, out, m, n, k, True, True, 1, False, alpha, None, None)
            return out
        out.zero_()
    ext().gemm(a, b, out, m, n, k, True, True, splits, True, alpha, None, None)
    return out


# --------------------------------------------------------------------------------------------------
# Linear
# --------------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Tensor | None):
        w16 = bf16_weight(weight)
        x16 = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        x2 = _gemm_ready(_as_2d(x16))
        y = matmul_nt(x2, w16)
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        ctx.x_dtype = x.dtype
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy: Tensor):
        x2, weight = ctx.saved_tensors
        dy2 = _gemm_ready(_as_2d(dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16)))
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = matmul_nn(dy2, bf16_weight(weight)).view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = matmul_tn(dy2, x2)
            if dw.dtype != weight.dtype:
                dw = dw.to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0)
        return dx, dw, db


class _FanoutLinearFn(torch.autograd.Function):
    """Several bias-free linears of one input. The backward pass chains the input-gradient GEMMs
    through the GEMM's residual epilogue (``dx = dy_i @ W_i + dx``) instead of leaving autograd to
    add one full-size gradient per branch with separate element-wise kernels."""

    @staticmethod
    def forward(ctx, x: Tensor, *weights: Tensor):
        x16 = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        x2 = _gemm_ready(_as_2d(x16))
        outs = tuple(matmul_nt(x2, bf16_weight(w)).view(*x.shape[:-1], w.shape[0]) for w in weights)
        ctx.save_for_backward(x2, *weights)
        ctx.x_shape = x.shape
        ctx.x_dtype = x.dtype
        return outs

    @staticmethod
    def backward(ctx, *dys: Tensor):
        x2, *weights = ctx.saved_tensors
        ready = [None if dy is None else _gemm_ready(_as_2d(
            dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16))) for dy in dys]
        dx = None
        if ctx.needs_input_grad[0]:
            for dy2, weight in zip(ready, weights):
                if dy2 is None:
                    continue
                w16 = _gemm_ready(bf16_weight(weight))
                m, k = dy2.shape
                n = w16.shape[-1]
                if dx is None:
                    dx = torch.empty((m, n), device=dy2.device, dtype=torch.bfloat16)
                    ext().gemm(dy2, w16, dx, m, n, k, False, True, 1, False, 1.0, None, None)
                else:  # in place: every element is read by the thread that then overwrites it
                    ext().gemm(dy2, w16, dx, m, n, k, False, True, 1, False, 1.0, None, None,
                               dx, 1.0)
            if dx is not None:
                dx = dx.view(ctx.x_shape)
                if dx.dtype != ctx.x_dtype:
                    dx = dx.to(ctx.x_dtype)
        dws = []
        for i, (dy2, weight) in enumerate(zip(ready, weights)):
            dw = None
            if dy2 is not None and ctx.needs_input_grad[1 + i]:
                dw = matmul_tn(dy2, x2)
                if dw.dtype != weight.dtype:
                    dw = dw.to(weight.dtype)
            dws.append(dw)
        return (dx, *dws)


def linear_fanout(x: Tensor, weights) -> tuple[Tensor, ...]:
    """``tuple(x @ w.T for w in weights)``: the projections that share an input (query / key /
    value; gate / up), with a fused input-gradient accumulation on the bf16 fast path."""
    weights = tuple(weights)
    if (fast_path(x) and x.shape[-1] % 8 == 0 and all(w.shape[0] % 8 == 0 for w in weights)
            and len(weights) > 1):
        return _FanoutLinearFn.apply(x, *weights)
    return tuple(linear(x, w) for w in weights)


def fused_projections(x: Tensor) -> bool:
    """Whether projections that share the input ``x`` should run as one GEMM (the bf16 fast path;
    ``OHARA_FUSED_PROJECTIONS=0`` keeps them separate, for A/B measurements)."""
    return _FUSE_PROJECTIONS and fast_path(x) and x.shape[-1] % 8 == 0


def fused_bf16_weight(weights) -> Tensor:
    """One contiguous ``(sum of out_features, in_features)`` bf16 matrix made of the compute copies
    of several weights that multiply the same input.

    When the copies already sit next to each other in memory (the first call makes it so) this is
    a zero-copy view; otherwise they are concatenated into a new buffer and every parameter's
    compute copy is re-pointed at its rows of that buffer, so that optimizers that refresh the
    copies in place keep the fused matrix current. A sharded optimizer re-points the copies at
    its own gathered buffer after every step; then the concatenation is repeated (a few MB)."""
    shadows = [bf16_weight(w) for w in weights]
    first = shadows[0]
    cols = first.shape[1]
    rows = sum(s.shape[0] for s in shadows)
    storage = first.untyped_storage().data_ptr()
    expected = first.data_ptr()
    adjacent = True
    for shadow in shadows:
        if (shadow.shape[1] != cols or not shadow.is_contiguous()
                or shadow.untyped_storage().data_ptr() != storage
                or shadow.data_ptr() != expected):
            adjacent = False
            break
        expected += shadow.numel() * 2
    if adjacent:
        return first.as_strided((rows, cols), (cols, 1))
    fused = torch.cat(shadows, dim=0)
    begin = 0
    for weight, shadow in zip(weights, shadows):
        end = begin + shadow.shape[0]
        if weight.dtype != torch.bfloat16:  # a bf16 parameter is its own compute copy
            refresh_bf16_weight(weight, fused[begin:end])
        begin = end
    return fused


class _LinearCatFn(torch.autograd.Function):
    """``x @ concat(weights).T`` as ONE product: a single wide GEMM forward, a single
    input-gradient GEMM with the long reduction (instead of one residual-chained GEMM per
    weight) and a single weight-gradient GEMM whose row blocks are the gradients of the
    individual weights."""

    @staticmethod
    def forward(ctx, x: Tensor, *weights: Tensor):
        x16 = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        x2 = _gemm_ready(_as_2d(x16))
        y = matmul_nt(x2, fused_bf16_weight(weights))
        ctx.save_for_backward(x2, *weights)
        ctx.x_shape = x.shape
        ctx.x_dtype = x.dtype
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy: Tensor):
        x2, *weights = ctx.saved_tensors
        dy2 = _gemm_ready(_as_2d(dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16)))
        dx = None
        if ctx.needs_input_grad[0]:
            dx = matmul_nn(dy2, fused_bf16_weight(weights)).view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        grads: list[Tensor | None] = [None] * len(weights)
        if any(ctx.needs_input_grad[1:]):
            dw = matmul_tn(dy2, x2)  # (sum of out_features, in_features) fp32
            begin = 0
            for i, weight in enumerate(weights):
                end = begin + weight.shape[0]
                if ctx.needs_input_grad[1 + i]:
                    part = dw[begin:end]
                    grads[i] = part if part.dtype == weight.dtype else part.to(weight.dtype)
                begin = end
        return (dx, *grads)


def linear_cat(x: Tensor, weights) -> Tensor:
    """``concat([x @ w.T for w in weights], dim=-1)`` — the projections that share an input
    (query | key | value; gate | up) — computed as one GEMM on the bf16 fast path. The consumers
    (:func:`rope_attention`, :func:`swiglu_cat`) read their operands as column slices of the
    result and return one gradient for all of it."""
    weights = tuple(weights)
    if (fast_path(x) and x.shape[-1] % 8 == 0 and all(w.shape[0] % 8 == 0 for w in weights)):
        return _LinearCatFn.apply(x, *weights)
    return torch.cat([F.linear(x, w) for w in weights], dim=-1)


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    """``x @ weight.T + bias`` with the tcgen05 GEMM on the bf16 fast path."""
    if fast_path(x) and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
        return _LinearFn.apply(x, weight, bias)
    return F.linear(x, weight, bias)


# --------------------------------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, eps: float):
        x16 = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
        w32 = _f32_weight(weight)
        y, rstd = ext().rmsnorm_fwd(x16, None, w32, eps)
        ctx.save_for_backward(x16, w32, rstd)
        ctx.x_dtype = x.dtype
        ctx.w_dtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):
        x16, w32, rstd = ctx.saved_tensors
        dy16 = (dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16)).contiguous()
        dx, dw = ext().rmsnorm_bwd(dy16, x16, w32, rstd, None)
        return dx.to(ctx.x_dtype), dw.to(ctx.w_dtype), None


class _AddRMSNormFn(torch.autograd.Function):
    """``s = x + delta; y = rms_norm(s)`` in one kernel; backward folds the residual gradient
    into the norm backward (``ds = norm_bwd(dy) + d_s``), so neither add is a separate pass."""

    @staticmethod
    def forward(ctx, x: Tensor, delta: Tensor, weight: Tensor, eps: float):
        x16 = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
        d16 = (delta if delta.dtype == torch.bfloat16 else delta.to(torch.bfloat16)).contiguous()
        w32 = _f32_weight(weight)
        y, rstd, summed = ext().rmsnorm_fwd(x16, d16, w32, eps)
        ctx.save_for_backward(summed, w32, rstd)
        ctx.dtypes = (x.dtype, delta.dtype, weight.dtype)
        return y, summed

    @staticmethod
    def backward(ctx, dy: Tensor, dsum: Tensor | None):
        summed, w32, rstd = ctx.saved_tensors
        dy16 = (dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16)).contiguous()
        if dsum is not None:
            dsum = (dsum if dsum.dtype == torch.bfloat16 else dsum.to(torch.bfloat16)).contiguous()
        ds, dw = ext().rmsnorm_bwd(dy16, summed, w32, rstd, dsum)
        return ds.to(ctx.dtypes[0]), ds.to(ctx.dtypes[1]), dw.to(ctx.dtypes[2]), None


def add_rms_norm(x: Tensor, delta: Tensor | None, weight: Tensor,
                 eps: float = 1e-5) -> tuple[Tensor, Tensor]:
    """Return ``(rms_norm(x + delta), x + delta)``; ``delta=None`` means no residual to add."""
    if delta is None:
        return rms_norm(x, weight, eps), x
    if fast_path(x) and x.shape[-1] % 8 == 0 and x.shape == delta.shape:
        return _AddRMSNormFn.apply(x, delta, weight, eps)
    summed = x + delta.to(x.dtype)
    return rms_norm(summed, weight, eps), summed


def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-5) -> Tensor:
    if fast_path(x) and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, weight, eps)
    from ohara_b200.modules.norm import rms_norm_reference

    return rms_norm_reference(x, weight, eps)


# --------------------------------------------------------------------------------------------------
# RoPE
# --------------------------------------------------------------------------------------------------
class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, cos: Tensor, sin: Tensor):
        ctx.save_for_backward(cos, sin)
        ctx.dtypes = (q.dtype, k.dtype)
        q16 = q if q.dtype == torch.bfloat16 else q.to(torch.bfloat16)
        k16 = k if k.dtype == torch.bfloat16 else k.to(torch.bfloat16)
        qo, ko = ext().rope(q16, k16, cos, sin, False)
        return qo, ko

    @staticmethod
    def backward(ctx, dq: Tensor, dk: Tensor):
        cos, sin = ctx.saved_tensors
        dq16 = dq if dq.dtype == torch.bfloat16 else dq.to(torch.bfloat16)
        dk16 = dk if dk.dtype == torch.bfloat16 else dk.to(torch.bfloat16)
        gq, gk = ext().rope(dq16, dk16, cos, sin, True)
        return gq.to(ctx.dtypes[0]), gk.to(ctx.dtypes[1]), None, None


def rope_qk(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor) -> tuple[Tensor, Tensor]:
    """Interleaved-pair rotary embedding of q and k, ``(B, T, H, D)``, one launch for both."""
    if fast_path(q) and q.shape[-1] % 8 == 0:
        seq = q.shape[1]
        cos = cos[:seq].float().contiguous()
        sin = sin[:seq].float().contiguous()
        return _RopeFn.apply(q, k, cos, sin)
    from ohara_b200.embeddings_pos.rotary import rope_reference

    return rope_reference(q, cos, sin), rope_reference(k, cos, sin).to(q.dtype)


# --------------------------------------------------------------------------------------------------
# SwiGLU
# --------------------------------------------------------------------------------------------------
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate: Tensor, up: Tensor):
        g2, u2 = _as_2d(gate), _as_2d(up)
        a = ext().swiglu_fwd(g2, u2)
        ctx.save_for_backward(g2, u2)
        ctx.shape = gate.shape
        return a.view(gate.shape)

    @staticmethod
    def backward(ctx, da: Tensor):
        g2, u2 = ctx.saved_tensors
        da2 = _as_2d(da.contiguous())
        dg = torch.empty_like(g2, memory_format=torch.contiguous_format)
        du = torch.empty_like(u2, memory_format=torch.contiguous_format)
        ext().swiglu_bwd(da2, g2, u2, dg, du)
        return dg.view(ctx.shape), du.view(ctx.shape)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """``silu(gate) * up`` in one pass (and one pass backward)."""
    if (
        gate.is_cuda
        and gate.dtype == torch.bfloat16
        and up.dtype == torch.bfloat16
        and gate.shape[-1] % 8 == 0
    ):
        return _SwiGLUFn.apply(gate.contiguous(), up.contiguous())
    return F.silu(gate) * up


class _SwiGLUCatFn(torch.autograd.Function):
    """``silu(gu[:, :h]) * gu[:, h:]`` on the two column halves of one matrix; the backward pass
    writes both gradients into the halves of one buffer, which is the gradient of ``gu``."""

    @staticmethod
    def forward(ctx, gu: Tensor):
        gu2 = _as_2d(gu)
        half = gu2.shape[1] // 2
        a = ext().swiglu_fwd(gu2[:, :half], gu2[:, half:])
        ctx.save_for_backward(gu2)
        ctx.shape = gu.shape
        return a.view(*gu.shape[:-1], half)

    @staticmethod
    def backward(ctx, da: Tensor):
        (gu2,) = ctx.saved_tensors
        half = gu2.shape[1] // 2
        da2 = _as_2d(da.contiguous())
        dgu = torch.empty_like(gu2, memory_format=torch.contiguous_format)
        ext().swiglu_bwd(da2, gu2[:, :half], gu2[:, half:], dgu[:, :half], dgu[:, half:])
        return dgu.view(ctx.shape)


def swiglu_cat(gu: Tensor) -> Tensor:
    """SwiGLU of a fused ``gate | up`` projection: ``silu(gu[..., :h]) * gu[..., h:]``."""
    half = gu.shape[-1] // 2
    if (gu.is_cuda and gu.dtype == torch.bfloat16 and half % 8 == 0 and gu.shape[-1] == 2 * half
            and gu.is_contiguous()):
        return _SwiGLUCatFn.apply(gu)
    return F.silu(gu[..., :half]) * gu[..., half:]


# --------------------------------------------------------------------------------------------------
# Embedding
# --------------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids: Tensor, table: Tensor):
        ctx.save_for_backward(ids)
        ctx.table_shape = table.shape
        return ext().embedding_fwd(ids.contiguous(), table.detach())

    @staticmethod
    def backward(ctx, dout: Tensor):
        (ids,) = ctx.saved_tensors
        dtable = torch.zeros(ctx.table_shape, device=dout.device, dtype=torch.float32)
        ext().embedding_bwd(ids.contiguous(), dout.contiguous(), dtable)
        return None, dtable


def embedding(ids: Tensor, table: Tensor) -> Tensor:
    """Row gather; on the fast path reads the fp32 table and emits bf16 activations directly."""
    if (
        fast_path(table)
        and table.dtype == torch.float32
        and table.is_contiguous()
        and table.shape[1] % 8 == 0
        and ids.dtype == torch.int64
    ):
        return _EmbeddingFn.apply(ids, table)
    return F.embedding(ids, table)


# --------------------------------------------------------------------------------------------------
# Attention (implemented in ops/attention.py) and fused linear + cross-entropy (ops/loss.py)
# --------------------------------------------------------------------------------------------------
from .attention import attention, rope_attention  # noqa: E402
from .loss import linear_cross_entropy  # noqa: E402
