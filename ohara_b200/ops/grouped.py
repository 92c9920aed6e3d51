"""Grouped (per-expert) GEMMs for mixture-of-experts layers on the tcgen05 kernel.

Tokens routed to expert ``e`` occupy a contiguous row group of a padded buffer; every group starts
on a multiple of ``TILE`` rows (the height of a GEMM pair tile), so each tile belongs to exactly one expert and the
kernel picks the weight matrix from a per-tile expert table. Nothing here synchronises with the
host: buffer sizes are static upper bounds (``pairs + experts * TILE`` rows).
"""

from __future__ import annotations

import torch
from torch import Tensor

from ohara_b200.utils.checks import debug_checks_enabled, validate_dispatch_plan

from ._ext import ext

_DEBUG_CHECKS = debug_checks_enabled()
TILE = 256  # rows every expert segment is padded to: one CTA-pair tile of the grouped GEMM


def build_dispatch_plan(expert_indices: Tensor, num_experts: int):
    """Sort (token, expert) pairs by expert and lay them out in a tile-padded buffer.

    Returns ``(token_of_row, dest_row, order, tile_expert, k_offsets, padded_rows)`` where
    ``dest_row[j]`` is the padded row of the j-th sorted pair, ``tile_expert[t]`` the expert of
    ``TILE``-row tile ``t`` (−1 for unused tiles) and ``k_offsets`` the (E+1) padded group boundaries.
    """
    tokens, k = expert_indices.shape
    pairs = tokens * k
    flat = expert_indices.reshape(-1)
    order = torch.argsort(flat, stable=True)
    token_of_row = order.div(k, rounding_mode="floor")
    counts = torch.bincount(flat, minlength=num_experts)
    padded_counts = (counts + (TILE - 1)) // TILE * TILE
    padded_ends = padded_counts.cumsum(0)
    padded_starts = padded_ends - padded_counts
    starts = counts.cumsum(0) - counts
    sorted_expert = flat[order]
    rank_in_expert = torch.arange(pairs, device=flat.device) - starts[sorted_expert]
    dest_row = padded_starts[sorted_expert] + rank_in_expert
    padded_rows = (pairs + num_experts * (TILE - 1)) // TILE * TILE + TILE
    num_tiles = padded_rows // TILE
    tile_begin = torch.arange(num_tiles, device=flat.device) * TILE
    tile_expert = torch.searchsorted(padded_ends, tile_begin, right=True)
    tile_expert = torch.where(tile_begin < padded_ends[-1], tile_expert, -1).to(torch.int32)
    # Rows of expert e: [padded_start[e], padded_start[e] + padded_count[e]); zero padding rows
    # contribute nothing to the weight gradient.
    k_offsets = torch.cat([padded_starts[:1], padded_ends]).to(torch.int32)
    return token_of_row, dest_row, order, tile_expert, k_offsets, padded_rows


class _GroupedLinearFn(torch.autograd.Function):
    """``y[rows of expert e] = x[rows of expert e] @ w[e]`` with ``w (E, in, out)``."""

    @staticmethod
    def forward(ctx, x_pad: Tensor, weight: Tensor, tile_expert: Tensor, k_offsets: Tensor,
                out=None):
        from . import bf16_weight

        w16 = bf16_weight(weight)
        rows, k = x_pad.shape
        n = weight.shape[2]
        # ``out``: a callable that returns a caller-owned (rows, n) bf16 buffer, e.g. symmetric
        # memory that peers read. It is called here, inside the function, so that the buffer is
        # not an input of the autograd node (an input written in place and returned would make
        # autograd copy it back through its base in the backward pass).
        y = out() if out is not None else torch.empty(rows, n, device=x_pad.device,
                                                      dtype=torch.bfloat16)
        # B[e] stored (K=in rows, N=out contiguous): MN-major.
        ext().gemm(x_pad, w16, y, rows, n, k, False, True, 1, False, 1.0, tile_expert, None,
                   None, 1.0, TILE)
        ctx.save_for_backward(x_pad, weight, tile_expert, k_offsets)
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):
        from . import bf16_weight

        x_pad, weight, tile_expert, k_offsets = ctx.saved_tensors
        dy = dy.contiguous()
        rows, k = x_pad.shape
        experts, _, n = weight.shape
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x_pad)
            # dx = dy @ w[e]^T: B[e] as (N'=in rows, K'=out contiguous): K-major.
            ext().gemm(dy, bf16_weight(weight), dx, rows, k, n, False, False, 1, False, 1.0,
                       tile_expert, None, None, 1.0, TILE)
        if ctx.needs_input_grad[1]:
            # every (expert, tile) of dw is written by the kernel, zeros for an expert without rows
            dw = torch.empty(experts, k, n, device=dy.device, dtype=torch.float32)
            # dw[e] = x_e^T @ dy_e: both operands MN-major over the expert's token range.
            ext().gemm(x_pad, dy, dw, k, n, rows, True, True, 1, False, 1.0, None, k_offsets)
            if dw.dtype != weight.dtype:
                dw = dw.to(weight.dtype)
        return dx, dw, None, None, None


def grouped_linear(x_pad: Tensor, weight: Tensor, tile_expert: Tensor, k_offsets: Tensor,
                   out=None) -> Tensor:
    return _GroupedLinearFn.apply(x_pad, weight, tile_expert, k_offsets, out)


def grouped_swiglu_experts(flat_x: Tensor, expert_indices: Tensor, expert_weights: Tensor,
                           w_gate: Tensor, w_up: Tensor, w_down: Tensor,
                           counts: Tensor | None = None) -> Tensor:
    """Routed SwiGLU experts: permute -> 3 grouped GEMMs (+ fused activation) -> weighted combine.
    ``counts`` (tokens per expert, int32) comes for free from the routing kernel; without it the
    indices are counted here."""
    from . import moe, swiglu

    num_experts = w_gate.shape[0]
    k = expert_indices.shape[1]
    x16 = flat_x if flat_x.dtype == torch.bfloat16 else flat_x.to(torch.bfloat16)
    indices = expert_indices if expert_indices.dtype == torch.int32 else expert_indices.int()
    if counts is None:
        counts = torch.bincount(indices.reshape(-1), minlength=num_experts).int()
    dest_row, row_pair, tile_expert, k_offsets = moe.dispatch_plan(indices, counts)
    if _DEBUG_CHECKS:  # OHARA_DEBUG_CHECKS=1: read the tables back and verify them (synchronises)
        validate_dispatch_plan(indices, dest_row, row_pair, tile_expert, k_offsets, TILE)
    x_pad = moe.permute_rows(x16, dest_row, row_pair, k)
    gate = grouped_linear(x_pad, w_gate, tile_expert, k_offsets)
    up = grouped_linear(x_pad, w_up, tile_expert, k_offsets)
    hidden = swiglu(gate, up)
    y_pad = grouped_linear(hidden, w_down, tile_expert, k_offsets)
    return moe.combine_rows(y_pad, expert_weights, dest_row, row_pair)
