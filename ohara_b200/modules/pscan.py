"""Parallel scan for first-order linear recurrences ``h[t] = a[t] * h[t-1] + x[t]`` (``h[-1] = 0``).

Used by Mamba's selective scan and the RG-LRU. The reference carries a Blelloch up/down-sweep
(ohara/modules/pscan.py:63-258). Here CUDA tensors run the one-pass kernels of ``csrc/pscan.cu``
(a thread owns four channels and walks the sequence; every tensor crosses HBM once, forward and
backward); fp32 CPU tensors run the same one-pass recurrence in the extension's host kernel
(``csrc/cpu_scan.cpp``) when the extension is built; other tensors use the Hillis-Steele doubling
form below, which needs ``ceil(log2 L)``
passes of whole-tensor operations, no padding to a power of two and no in-place tricks. Both have
an explicit backward that is itself a (reversed) scan:

    dx[t] = dh[t] + a[t+1] * dx[t+1]        da[t] = dx[t] * h[t-1]
"""

from __future__ import annotations

import torch
from torch import Tensor


def _scan_forward(a: Tensor, x: Tensor) -> Tensor:
    """Inclusive scan along dim 1 of ``(B, L, ...)`` tensors."""
    length = a.shape[1]
    coeff, value = a, x
    shift = 1
    while shift < length:
        # Compose element t with element t - shift: (c2, v2) o (c1, v1) = (c1*c2, c2*v1 + v2).
        prev_value = torch.zeros_like(value)
        prev_value[:, shift:] = value[:, :-shift]
        prev_coeff = torch.ones_like(coeff)
        prev_coeff[:, shift:] = coeff[:, :-shift]
        value = coeff * prev_value + value
        coeff = coeff * prev_coeff
        shift *= 2
    return value


class PScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a: Tensor, x: Tensor) -> Tensor:
        h = _scan_forward(a, x)
        ctx.save_for_backward(a, h)
        return h

    @staticmethod
    def backward(ctx, grad_h: Tensor):
        a, h = ctx.saved_tensors
        # Reverse-time recurrence with the coefficient of the *next* step.
        a_next = torch.zeros_like(a)
        a_next[:, :-1] = a[:, 1:]
        dx = _scan_forward(a_next.flip(1), grad_h.flip(1)).flip(1)
        h_prev = torch.zeros_like(h)
        h_prev[:, 1:] = h[:, :-1]
        return dx * h_prev, dx


class PScanCuda(torch.autograd.Function):
    """The same recurrence on the one-pass CUDA kernels; computes in fp32 whatever the input type."""

    @staticmethod
    def forward(ctx, a: Tensor, x: Tensor) -> Tensor:
        from ohara_b200.ops._ext import ext

        a32, x32 = a.float().contiguous(), x.float().contiguous()
        h = ext().pscan_fwd(a32, x32)
        ctx.save_for_backward(a32, h)
        ctx.dtypes = (a.dtype, x.dtype)
        return h.to(x.dtype)

    @staticmethod
    def backward(ctx, grad_h: Tensor):
        from ohara_b200.ops._ext import ext

        a32, h = ctx.saved_tensors
        da, dx = ext().pscan_bwd(a32, h, grad_h.float().contiguous())
        return da.to(ctx.dtypes[0]), dx.to(ctx.dtypes[1])


class PScanNative(torch.autograd.Function):
    """The recurrence on fp32 CPU tensors in one pass of the extension's host kernel
    (``csrc/cpu_scan.cpp``: a task owns a block of channels of one batch row and walks the
    sequence once), forward and backward."""

    @staticmethod
    def forward(ctx, a: Tensor, x: Tensor) -> Tensor:
        from ohara_b200.ops._ext import ext

        a32, x32 = a.contiguous(), x.contiguous()
        h = ext().pscan_cpu_fwd(a32, x32)
        ctx.save_for_backward(a32, h)
        return h

    @staticmethod
    def backward(ctx, grad_h: Tensor):
        from ohara_b200.ops._ext import ext

        a32, h = ctx.saved_tensors
        da, dx = ext().pscan_cpu_bwd(a32, h, grad_h.contiguous())
        return da, dx


_NATIVE_CPU: bool | None = None


def _native_cpu_scan() -> bool:
    """Whether the built extension is there to run CPU scans (never triggers a build: a CPU-only
    installation without the shared object uses the PyTorch form)."""
    global _NATIVE_CPU
    if _NATIVE_CPU is None:
        try:
            from ohara_b200 import build_ext
            from ohara_b200.ops import _ext

            _NATIVE_CPU = build_ext.ext_path().exists() and _ext.available() and hasattr(
                _ext.ext(), "pscan_cpu_fwd")
        except Exception:  # noqa: BLE001 - any failure to load means "use the PyTorch form"
            _NATIVE_CPU = False
    return _NATIVE_CPU


def npo2(len: int) -> int:  # noqa: A002 - the reference's parameter name
    """The smallest power of two that is at least ``len``."""
    return 1 << max(0, int(len) - 1).bit_length()


def pad_npo2(X: Tensor) -> Tensor:
    """Zero-pad dim 1 of ``(B, L, D, N)`` to the next power of two. Nothing here needs it (the
    scans take any length); kept because callers of the reference's scan pad with it
    (ohara/modules/pscan.py:39-60)."""
    extra = npo2(X.size(1)) - X.size(1)
    return torch.nn.functional.pad(X, (0, 0, 0, 0, 0, extra)) if extra else X


def pscan(A: Tensor, X: Tensor) -> Tensor:
    """``H`` with ``H[:, t] = A[:, t] * H[:, t-1] + X[:, t]`` for ``(B, L, D, N)`` (or any
    ``(B, L, ...)``) inputs of equal shape."""
    if A.shape != X.shape:
        raise ValueError("pscan expects coefficient and input tensors of the same shape")
    if A.is_cuda and X.is_cuda and A.dim() >= 2 and A.dtype != torch.float64:
        return PScanCuda.apply(A, X)
    if (not A.is_cuda and not X.is_cuda and A.dtype == torch.float32 and X.dtype == torch.float32
            and A.dim() >= 2 and _native_cpu_scan()):
        return PScanNative.apply(A, X)
    return PScan.apply(A, X)


def sequential_scan(A: Tensor, X: Tensor) -> Tensor:
    """Step-by-step oracle for :func:`pscan`."""
    h = torch.zeros_like(X[:, 0])
    out = []
    for t in range(X.shape[1]):
        h = A[:, t] * h + X[:, t]
        out.append(h)
    return torch.stack(out, dim=1)
