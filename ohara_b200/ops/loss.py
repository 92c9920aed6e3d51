"""Fused output projection + cross-entropy.

``linear_cross_entropy(hidden, weight, targets)`` returns ``scale * sum_i CE(hidden_i @ weight.T,
target_i)`` over targets that differ from ``ignore_index`` — the sum-reduction the trainer divides
by the number of supervised tokens (reference: ohara/trainer.py:464-478), so an assistant-only loss
mask is just ``ignore_index`` in ``targets``.

On CUDA the (tokens x vocab) logits are never materialised: tokens are processed in chunks; for
each chunk the tcgen05 GEMM writes bf16 logits, one kernel turns them in place into
``d loss / d logits`` while emitting the per-row loss, and two more GEMMs fold the chunk into the
hidden-state gradient and the (fp32, reduce-add) weight gradient. The backward pass therefore only
rescales by the incoming gradient.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from ._ext import ext


def linear_cross_entropy_reference(hidden: Tensor, weight: Tensor, targets: Tensor,
                                   ignore_index: int = -1, scale: Tensor | float | None = None) -> Tensor:
    logits = F.linear(hidden, weight).float()
    loss = F.cross_entropy(
        logits.reshape(-1, logits.size(-1)), targets.reshape(-1), ignore_index=ignore_index,
        reduction="sum",
    )
    return loss if scale is None else loss * scale


def _chunk_rows(tokens: int, vocab: int) -> int:
    # Keep one chunk of bf16 logits around 512 MiB: large enough to fill the machine with GEMM
    # tiles, small enough not to matter next to activations.
    budget = 512 * 1024 * 1024 // (2 * max(vocab, 1))
    rows = max(128, (budget // 128) * 128)
    return min(rows, max(128, ((tokens + 127) // 128) * 128))


class _LinearCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden: Tensor, weight: Tensor, targets: Tensor, ignore_index: int,
                scale: Tensor | None):
        from . import bf16_weight, matmul_nn, matmul_nt, matmul_tn

        C = ext()
        h2 = hidden.reshape(-1, hidden.shape[-1])
        if h2.dtype != torch.bfloat16:
            h2 = h2.to(torch.bfloat16)
        h2 = h2.contiguous()
        t1 = targets.reshape(-1).contiguous()
        tokens, dim = h2.shape
        vocab = weight.shape[0]
        w16 = bf16_weight(weight)
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        dh = torch.empty_like(h2) if need_dh else None
        dw = torch.zeros(vocab, dim, device=h2.device, dtype=torch.float32) if need_dw else None
        losses = torch.empty(tokens, device=h2.device, dtype=torch.float32)
        rows = _chunk_rows(tokens, vocab)
        pitch = (vocab + 7) // 8 * 8
        buf = torch.empty(rows, pitch, device=h2.device, dtype=torch.bfloat16)
        for start in range(0, tokens, rows):
            stop = min(start + rows, tokens)
            n = stop - start
            logits = buf[:n, :vocab]
            matmul_nt(h2[start:stop], w16, out=logits)
            loss_rows, _ = C.cross_entropy_rows(
                logits, t1[start:stop], scale, ignore_index, need_dh or need_dw, False
            )
            losses[start:stop] = loss_rows
            if need_dh:
                matmul_nn(logits, w16, out=dh[start:stop])
            if need_dw:
                matmul_tn(logits, h2[start:stop], out=dw, accumulate=True)
        total = losses.sum()
        if scale is not None:
            total = total * scale
        ctx.save_for_backward(dh, dw)
        ctx.hidden_shape = hidden.shape
        ctx.hidden_dtype = hidden.dtype
        ctx.weight_dtype = weight.dtype
        return total

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        dh, dw = ctx.saved_tensors
        C = ext()
        g = grad_out.detach().float().reshape(1).contiguous()
        if dh is not None:
            C.scale_by_scalar(dh, g)
            dh = dh.view(ctx.hidden_shape).to(ctx.hidden_dtype)
        if dw is not None:
            C.scale_by_scalar(dw, g)
            dw = dw.to(ctx.weight_dtype)
        return dh, dw, None, None, None


def linear_cross_entropy(hidden: Tensor, weight: Tensor, targets: Tensor, ignore_index: int = -1,
                         scale: Tensor | float | None = None) -> Tensor:
    """Sum of token cross-entropies of ``hidden @ weight.T`` against ``targets`` (times ``scale``)."""
    from . import fast_path

    if fast_path(hidden) and hidden.shape[-1] % 8 == 0:
        if scale is not None and not isinstance(scale, Tensor):
            scale = torch.tensor(float(scale), device=hidden.device, dtype=torch.float32)
        if scale is not None:
            scale = scale.detach().float().reshape(()).contiguous()
        return _LinearCEFn.apply(hidden, weight, targets, int(ignore_index), scale)
    return linear_cross_entropy_reference(hidden, weight, targets, ignore_index, scale)
