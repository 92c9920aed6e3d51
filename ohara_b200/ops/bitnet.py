"""BitNet b1.58 linear layer: ternary weights, int8 activations, straight-through gradients
(reference: experiments/bitnet/bitnet.py:29-57, two TorchScript quantisers around ``F.linear``).

``bit_linear(x, weight, norm_weight)`` computes

    xn = rms_norm(x, norm_weight)
    q  = clamp(round(xn * 127 / amax_row|xn|), -128, 127)          (int8 values per row)
    t  = clamp(round(weight / mean|weight|), -1, 1)                 (ternary values)
    y  = (q @ t^T) * (amax_row / 127) * mean|weight|  (+ bias)

and its gradients treat both roundings as the identity, which is what the reference's
``x + (quant(x) - x).detach()`` expressions do. ``q`` and ``t`` are small integers, exact in bf16,
so on a GPU the product runs on the bf16 tensor-core GEMM with fp32 accumulation and is exact; the
quantisers (with the norm fused into the activation one) and the re-scaling of the accumulators
are the kernels of ``csrc/quantize.cu``. The same function runs on CPU tensors with PyTorch
expressions in place of each kernel, which is how the gradient formulas are tested.
``activation_quant_reference`` / ``weight_quant_reference`` are the plain expressions of the
reference and the oracle of the tests.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from ._ext import ext


def activation_quant_reference(x: Tensor) -> Tensor:
    """Per-row int8 fake quantisation; the backward pass sees the identity."""
    scale = 127.0 / x.abs().amax(dim=-1, keepdim=True).clamp_min(1e-5)
    quantised = (x * scale).round().clamp(-128, 127) / scale
    return x + (quantised - x).detach()


def weight_quant_reference(w: Tensor) -> tuple[Tensor, Tensor]:
    """Ternary fake quantisation: the weight normalised to {-1, 0, 1} (with the straight-through
    gradient of ``w``) and the scale to multiply the product by."""
    inv = 1.0 / w.abs().mean().clamp_min(1e-5)
    ternary = (w * inv).round().clamp(-1, 1) / inv
    w_ste = w + (ternary - w).detach()
    scale = w_ste.abs().max().detach()
    return w_ste / scale, scale


def bit_linear_reference(x: Tensor, weight: Tensor, norm_weight: Tensor, bias: Tensor | None = None,
                         eps: float = 1e-5) -> Tensor:
    from ohara_b200.modules.norm import rms_norm_reference

    w, scale = weight_quant_reference(weight)
    out = F.linear(activation_quant_reference(rms_norm_reference(x, norm_weight, eps)), w) * scale
    return out if bias is None else out + bias


# -- the pieces, each a kernel on CUDA and a PyTorch expression elsewhere ----------------------------
def quantize_activations(x: Tensor, norm_weight: Tensor | None = None,
                         eps: float = 1e-5) -> tuple[Tensor, Tensor, Tensor | None]:
    """``(q, dequant, rstd)`` of a 2-D tensor: integer-valued ``q`` (same dtype as ``x``),
    ``dequant (rows,)`` fp32 with ``q * dequant[:, None]`` the fake-quantised rows, and, when
    ``norm_weight`` is given, the rows are RMS-normalised first and ``rstd`` is ``1 / rms``."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        weight32 = None if norm_weight is None else norm_weight.detach().float().contiguous()
        q, dequant, rstd = ext().bitnet_act_quant(x.contiguous(), weight32, eps)
        return q, dequant, (rstd if norm_weight is not None else None)
    rows = x.float()
    rstd = None
    if norm_weight is not None:
        rstd = torch.rsqrt(rows.pow(2).mean(-1) + eps)
        rows = rows * rstd[:, None] * norm_weight.float()
    amax = rows.abs().amax(dim=-1).clamp_min(1e-5)
    q = (rows * (127.0 / amax)[:, None]).round().clamp(-128, 127)
    return q.to(x.dtype), amax / 127.0, rstd


def quantize_weight(weight: Tensor) -> tuple[Tensor, Tensor]:
    """``(ternary, scale)``: values in {-1, 0, 1} (bf16 on CUDA) and ``scale (1,)`` fp32 =
    ``max(mean |weight|, 1e-5)``."""
    weight = weight.detach()
    if weight.is_cuda and weight.dtype in (torch.float32, torch.bfloat16):
        ternary, scale = ext().bitnet_weight_quant(weight.contiguous())
        return ternary, scale
    scale = weight.float().abs().mean().clamp_min(1e-5).reshape(1)
    ternary = (weight.float() * (1.0 / scale)).round().clamp(-1, 1)
    return ternary.to(weight.dtype), scale


def _on_kernels(x: Tensor, weight: Tensor) -> bool:
    # (the norm backward kernel handles rows of up to 8192 elements)
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0
            and weight.shape[1] % 8 == 0 and weight.shape[1] <= 8192)


class _BitLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, norm_weight: Tensor, bias: Tensor | None,
                eps: float) -> Tensor:
        from ohara_b200 import ops

        kernels = _on_kernels(x, weight)
        q, dequant, rstd = quantize_activations(x, norm_weight, eps)
        ternary, scale = quantize_weight(weight)
        if kernels:
            acc = ops.matmul_nt(q, ternary, out_dtype=torch.float32)
            bias32 = None if bias is None else bias.detach().float().contiguous()
            out = ext().bitnet_scale_rows(acc, dequant, scale, bias32)
        else:
            out = (q.float() @ ternary.float().t()) * dequant[:, None] * scale
            if bias is not None:
                out = out + bias.float()
            out = out.to(x.dtype)
        ctx.save_for_backward(x, norm_weight, rstd, q, dequant, ternary, scale)
        ctx.kernels = kernels
        ctx.has_bias = bias is not None
        ctx.dtypes = (weight.dtype, None if bias is None else bias.dtype)
        return out

    @staticmethod
    def backward(ctx, dy: Tensor):
        from ohara_b200 import ops

        x, norm_weight, rstd, q, dequant, ternary, scale = ctx.saved_tensors
        need_x, need_w, need_norm, need_bias = ctx.needs_input_grad[:4]
        dx = dw = dnorm = dbias = None
        if ctx.kernels:
            dy16 = (dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16)).contiguous()
            if need_x or need_norm:
                # through the rounding as the identity: d xn = (dy * scale) @ t
                d_normed = ops.matmul_nn(dy16, ternary, out_dtype=torch.float32)
                d_normed = (d_normed * scale).to(torch.bfloat16)
                dx, dnorm = ext().rmsnorm_bwd(d_normed, x, norm_weight.detach().float().contiguous(),
                                              rstd, None)
                dnorm = dnorm.to(norm_weight.dtype)
            if need_w:
                # d weight = dy^T @ (q * dequant): the row factor goes onto dy, q stays integral
                dw = ops.matmul_tn((dy16.float() * dequant[:, None]).to(torch.bfloat16), q)
                dw = dw.to(ctx.dtypes[0])
        else:
            dy32 = dy.float()
            if need_x or need_norm:
                d_normed = (dy32 @ ternary.float()) * scale
                x32, w32 = x.float(), norm_weight.float()
                dnorm = (d_normed * x32 * rstd[:, None]).sum(0).to(norm_weight.dtype)
                g = d_normed * w32
                dx = rstd[:, None] * (g - x32 * (rstd ** 2)[:, None] * (g * x32).mean(-1, keepdim=True))
                dx = dx.to(x.dtype)
            if need_w:
                dw = ((dy32 * dequant[:, None]).t() @ q.float()).to(ctx.dtypes[0])
        if ctx.has_bias and need_bias:
            dbias = dy.float().sum(0).to(ctx.dtypes[1])
        return (dx if need_x else None, dw, dnorm if need_norm else None, dbias, None)


def bit_linear(x: Tensor, weight: Tensor, norm_weight: Tensor, bias: Tensor | None = None,
               eps: float = 1e-5) -> Tensor:
    """BitNet b1.58 linear layer on ``x (..., in)`` with ``weight (out, in)`` and the weight
    ``(in,)`` of the RMS norm in front of the activation quantiser. bf16 CUDA inputs (or fp32 ones
    inside a bf16 autocast region) run the kernels; the result then is bf16."""
    from ohara_b200.ops import fast_path

    lead = x.shape[:-1]
    rows = x.reshape(-1, x.shape[-1])
    if fast_path(rows) and rows.dtype != torch.bfloat16:
        rows = rows.to(torch.bfloat16)
    out = _BitLinearFn.apply(rows.contiguous(), weight, norm_weight, bias, eps)
    return out.reshape(*lead, weight.shape[0])
