"""Mixture-of-experts routing and dispatch on the CUDA kernels of ``csrc/moe.cu``.

``router_logits`` keeps near-fp32 accuracy on the bf16 tensor cores by splitting the fp32 router
weight into a bf16 head and a bf16 remainder (two GEMMs accumulating into one fp32 output).
``route`` is the top-k(+1) kernel with gate weights, the balancing threshold and per-expert counts
in one launch; ``permute_rows`` / ``combine_rows`` move tokens to and from the tile-padded,
expert-contiguous buffer the grouped GEMM reads. Nothing here synchronises with the host.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ._ext import ext

TILE = 256  # rows every expert segment is padded to: one CTA-pair tile of the grouped GEMM


# --------------------------------------------------------------------------------------------------
# Router
# --------------------------------------------------------------------------------------------------
class _RouterLogitsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x16: Tensor, weight: Tensor) -> Tensor:
        w = weight.detach().float()
        head = w.to(torch.bfloat16)
        rest = (w - head.float()).to(torch.bfloat16)
        tokens, dim = x16.shape
        experts = weight.shape[0]
        out = torch.empty(tokens, experts, device=x16.device, dtype=torch.float32)
        ext().gemm(x16, head, out, tokens, experts, dim, False, False)
        ext().gemm(x16, rest, out, tokens, experts, dim, False, False, 1, True)
        ctx.save_for_backward(x16, head)
        ctx.weight_dtype = weight.dtype
        return out

    @staticmethod
    def backward(ctx, dlogits: Tensor):
        from . import matmul_nn, matmul_tn

        x16, head = ctx.saved_tensors
        d16 = dlogits.to(torch.bfloat16)
        dx = matmul_nn(d16, head) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = matmul_tn(d16, x16).to(ctx.weight_dtype)
        return dx, dw


def router_logits_supported(x: Tensor, weight: Tensor) -> bool:
    experts, dim = weight.shape
    return x.is_cuda and experts % 4 == 0 and dim % 8 == 0


def router_logits(x16: Tensor, weight: Tensor) -> Tensor:
    """fp32 ``x16 @ weight.T`` for bf16 activations ``(N, D)`` and an fp32 router weight ``(E, D)``."""
    return _RouterLogitsFn.apply(x16.contiguous(), weight)


class _RouteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: Tensor, bias: Tensor | None, k: int, gate_fn: str, normalize: bool,
                want_alpha: bool):
        counts = torch.zeros(logits.shape[1], device=logits.device, dtype=torch.int32)
        sigmoid = gate_fn == "sigmoid"
        indices, weights, alpha = ext().route_topk(logits, bias, k, sigmoid, sigmoid and normalize,
                                                   want_alpha, counts)
        ctx.save_for_backward(logits, indices, weights)
        ctx.sigmoid, ctx.normalize = sigmoid, sigmoid and normalize
        ctx.mark_non_differentiable(indices, alpha, counts)
        return indices, weights, alpha, counts

    @staticmethod
    def backward(ctx, d_indices, d_weights, d_alpha, d_counts):
        logits, indices, weights = ctx.saved_tensors
        index64 = indices.long()
        if ctx.sigmoid:
            gate = torch.sigmoid(logits.gather(-1, index64))
            if ctx.normalize:
                total = gate.sum(-1, keepdim=True).clamp_min(1e-9)
                d_gate = (d_weights - (d_weights * weights).sum(-1, keepdim=True)) / total
            else:
                d_gate = d_weights
            d_chosen = d_gate * gate * (1 - gate)
        else:
            d_chosen = weights * (d_weights - (d_weights * weights).sum(-1, keepdim=True))
        d_logits = torch.zeros_like(logits).scatter_add_(-1, index64, d_chosen)
        return d_logits, None, None, None, None, None


def route(logits: Tensor, bias: Tensor | None, k: int, gate_fn: str, normalize: bool,
          want_alpha: bool):
    """``(indices int32 (N,k), weights fp32 (N,k), alpha fp32 (N,) or empty, counts int32 (E,))``.
    Selection uses ``logits + bias``; weights use the raw logits of the chosen experts; ``alpha``
    is the (k+1)-th biased score."""
    return _RouteFn.apply(logits.contiguous(), bias, k, gate_fn, normalize, want_alpha)


def accumulate_quantile(logits: Tensor, alpha: Tensor, beta_sum: Tensor, rank: int) -> None:
    """``beta_sum[e] += rank-th largest of (logits[:, e] - alpha)``: the per-expert threshold at
    which the expert would receive exactly its fair share of tokens."""
    ext().qb_quantile(logits.contiguous(), alpha.contiguous().view(-1), beta_sum, rank)


# --------------------------------------------------------------------------------------------------
# Dispatch
# --------------------------------------------------------------------------------------------------
def dispatch_plan(indices: Tensor, counts: Tensor):
    """``(dest_row (N*k,), row_pair (rows,), tile_expert (rows/TILE,), k_offsets (E+1,))`` for int32
    ``indices (N, k)`` and the per-expert ``counts``; every expert segment starts on a ``TILE``-row
    boundary and ``rows`` is a static upper bound."""
    return ext().moe_plan(indices.contiguous(), counts, TILE)


class _PermuteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x16: Tensor, dest_row: Tensor, row_pair: Tensor, k: int) -> Tensor:
        x_pad = torch.empty(row_pair.numel(), x16.shape[1], device=x16.device, dtype=torch.bfloat16)
        ext().moe_scatter_rows(x16, dest_row, None, row_pair, x_pad, k)
        ctx.save_for_backward(dest_row)
        ctx.k = k
        return x_pad

    @staticmethod
    def backward(ctx, dx_pad: Tensor):
        (dest_row,) = ctx.saved_tensors
        dx, _ = ext().moe_gather_combine(dx_pad.contiguous(), dest_row, None, None, ctx.k, True)
        return dx, None, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_pad: Tensor, weights: Tensor, dest_row: Tensor, row_pair: Tensor) -> Tensor:
        k = weights.shape[1]
        weights = weights.contiguous()
        out, _ = ext().moe_gather_combine(y_pad, dest_row, weights, None, k, True)
        ctx.save_for_backward(y_pad, weights, dest_row, row_pair)
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        y_pad, weights, dest_row, row_pair = ctx.saved_tensors
        k = weights.shape[1]
        dout = dout.contiguous()
        dy_pad = dweights = None
        if ctx.needs_input_grad[0]:
            dy_pad = torch.empty_like(y_pad)
            ext().moe_scatter_rows(dout, dest_row, weights, row_pair, dy_pad, k)
        if ctx.needs_input_grad[1]:
            _, dweights = ext().moe_gather_combine(y_pad, dest_row, None, dout, k, False)
        return dy_pad, dweights, None, None


def permute_rows(x16: Tensor, dest_row: Tensor, row_pair: Tensor, k: int) -> Tensor:
    """Copy token ``t`` to the padded rows of its ``k`` (token, expert) pairs; padding rows are 0."""
    return _PermuteFn.apply(x16.contiguous(), dest_row, row_pair, k)


def combine_rows(y_pad: Tensor, weights: Tensor, dest_row: Tensor, row_pair: Tensor) -> Tensor:
    """``out[t] = sum_i weights[t, i] * y_pad[row of pair (t, i)]`` in bf16 (fp32 accumulation)."""
    return _CombineFn.apply(y_pad.contiguous(), weights.float(), dest_row, row_pair)
