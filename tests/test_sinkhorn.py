"""Sinkhorn normalisation: the PyTorch expression on CPU (properties) and, on a GPU, the
register-resident and block-resident kernels against it (values and gradients)."""

import pytest
import torch

from ohara_b200.ops.sinkhorn import sinkhorn_log, sinkhorn_reference


def test_reference_is_doubly_stochastic_and_shift_invariant():
    torch.manual_seed(0)
    x = torch.randn(5, 7, 4, 4) * 3
    out = sinkhorn_log(x, iters=200)
    # the last half-step normalises the columns exactly; the rows converge
    assert torch.allclose(out.sum(-2), torch.ones(5, 7, 4), atol=1e-5)
    assert torch.allclose(out.sum(-1), torch.ones(5, 7, 4), atol=1e-2)
    assert torch.allclose(sinkhorn_log(x + 11.0, iters=200), out, atol=1e-5)
    with pytest.raises(ValueError):
        sinkhorn_log(torch.randn(3, 4, 5))


@pytest.mark.gpu
@pytest.mark.parametrize("n,iters", [(2, 5), (3, 12), (4, 20), (4, 1), (5, 8), (8, 20), (16, 10),
                                     (33, 6), (64, 12)])
def test_kernel_matches_reference_values_and_gradients(n, iters):
    torch.manual_seed(1)
    count = 129 if n <= 8 else 17
    x = (torch.randn(3, count, n, n, device="cuda") * 2).requires_grad_()
    w = torch.randn(3, count, n, n, device="cuda")
    out = sinkhorn_log(x, iters)
    (out * w).sum().backward()
    xr = x.detach().double().requires_grad_()
    ref = sinkhorn_reference(xr, iters)
    (ref * w.double()).sum().backward()
    assert torch.allclose(out.double(), ref, atol=2e-5)
    assert torch.allclose(x.grad.double(), xr.grad, atol=2e-4), (x.grad.double() - xr.grad).abs().max()


@pytest.mark.gpu
def test_matrices_beyond_the_kernels_fall_back_to_the_expression():
    x = torch.randn(4, 80, 80, device="cuda")
    assert torch.allclose(sinkhorn_log(x, 10), sinkhorn_reference(x, 10), atol=1e-6)
