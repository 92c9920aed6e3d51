"""Low-rank approximation via truncated SVD (reference: ohara/utils/svd.py:6-31)."""

from __future__ import annotations

import torch


def svd_approx(W: torch.Tensor, r: int | None = None):
    """Return ``(A, B, rank, error)`` with ``A @ B ≈ W`` of rank ``r`` and the Frobenius error."""
    U, S, Vh = torch.linalg.svd(W, full_matrices=False)
    r = S.size(0) if r is None else min(r, S.size(0))
    A = U[:, :r]
    B = torch.diag(S[:r]) @ Vh[:r, :]
    return A, B, r, torch.linalg.norm(W - A @ B)
