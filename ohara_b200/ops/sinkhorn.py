"""Log-domain Sinkhorn normalisation (doubly stochastic mixing matrices of manifold
hyper-connections; reference: experiments/mHC/sinkhorn.py:15-20 and its Triton kernels :59-200).

``sinkhorn_log(log_alpha, iters)``: subtract the maximum of each matrix, then ``iters`` times
subtract the row log-sum-exp and the column log-sum-exp, and return ``exp`` of the result. CUDA
tensors run the kernels of ``csrc/sinkhorn.cu`` (forward and an exact vector-Jacobian product):
matrices of 2 to 4 rows live in the registers of one thread, matrices of 5 to 64 rows (the range of
the reference's fused Triton kernel) in the shared memory of one block. Everything else runs the
PyTorch expression below, which is also the oracle of the kernels' tests.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ._ext import ext


def sinkhorn_reference(log_alpha: Tensor, iters: int) -> Tensor:
    x = log_alpha - log_alpha.amax(dim=(-2, -1), keepdim=True)
    for _ in range(iters):
        x = x - torch.logsumexp(x, dim=-1, keepdim=True)
        x = x - torch.logsumexp(x, dim=-2, keepdim=True)
    return torch.exp(x)


class _SinkhornFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, log_alpha: Tensor, iters: int) -> Tensor:
        x = log_alpha.float().contiguous()
        ctx.save_for_backward(x)
        ctx.iters = iters
        ctx.dtype = log_alpha.dtype
        return ext().sinkhorn_fwd(x, iters).to(log_alpha.dtype)

    @staticmethod
    def backward(ctx, grad: Tensor):
        (x,) = ctx.saved_tensors
        grad_in = ext().sinkhorn_bwd(x, grad.float().contiguous(), ctx.iters)
        return grad_in.to(ctx.dtype), None


def sinkhorn_log(log_alpha: Tensor, iters: int = 20, eps: float = 1e-6) -> Tensor:
    """``eps`` is accepted for signature parity with the reference, which does not use it either."""
    if log_alpha.dim() < 2 or log_alpha.shape[-1] != log_alpha.shape[-2]:
        raise ValueError("sinkhorn_log expects square matrices in the last two dimensions")
    if log_alpha.is_cuda and ext().sinkhorn_supported(log_alpha.shape[-1], iters):
        return _SinkhornFn.apply(log_alpha, iters)
    return sinkhorn_reference(log_alpha.float(), iters).to(log_alpha.dtype)
