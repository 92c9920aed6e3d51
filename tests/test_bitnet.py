"""BitNet b1.58 layer: the function with hand-written gradients (the form the GPU kernels use)
against autograd through the reference's straight-through expressions."""

import pytest
import torch

from ohara_b200.ops.bitnet import (activation_quant_reference, bit_linear, bit_linear_reference,
                                   quantize_activations, quantize_weight, weight_quant_reference)


def test_quantisers_split_into_integers_and_scales():
    torch.manual_seed(0)
    x = torch.randn(7, 32) * 3
    q, dequant, rstd = quantize_activations(x)
    assert rstd is None and torch.equal(q, q.round()) and q.abs().max() <= 128
    assert int(q.abs().amax(dim=-1).min()) == 127          # every row uses its full range
    torch.testing.assert_close(q * dequant[:, None], activation_quant_reference(x))

    w = torch.randn(24, 32)
    ternary, scale = quantize_weight(w)
    assert set(ternary.unique().tolist()) <= {-1.0, 0.0, 1.0} and scale.shape == (1,)
    normalised, reference_scale = weight_quant_reference(w)
    torch.testing.assert_close(ternary, normalised)
    torch.testing.assert_close(scale[0], reference_scale)

    zeros, zero_scale = quantize_weight(torch.zeros(4, 8))
    assert float(zero_scale) == pytest.approx(1e-5) and not zeros.any()


@pytest.mark.parametrize("bias", [False, True])
def test_bit_linear_matches_autograd_through_the_reference_expressions(bias):
    torch.manual_seed(1)
    x = torch.randn(3, 5, 64, requires_grad=True)
    weight = torch.randn(48, 64, requires_grad=True)
    norm_weight = torch.empty(64).uniform_(0.5, 1.5).requires_grad_()
    b = torch.randn(48, requires_grad=True) if bias else None
    grad = torch.randn(3, 5, 48)
    inputs = [t for t in (x, weight, norm_weight, b) if t is not None]

    want = bit_linear_reference(x, weight, norm_weight, b)
    want_grads = torch.autograd.grad(want, inputs, grad)
    got = bit_linear(x, weight, norm_weight, b)
    got_grads = torch.autograd.grad(got, inputs, grad)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    for have, ref in zip(got_grads, want_grads):
        torch.testing.assert_close(have, ref, rtol=1e-4, atol=1e-4)


def test_bitlinear_module_trains_and_replaces_linears():
    from experiments.bitnet.bitnet import BitLinear, apply_bitlinear

    torch.manual_seed(2)
    net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    net = apply_bitlinear(net)
    assert sum(isinstance(m, BitLinear) for m in net.modules()) == 2
    optimizer = torch.optim.Adam(net.parameters(), lr=1e-2)
    x, y = torch.randn(64, 16), torch.randint(0, 4, (64,))
    losses = []
    for _ in range(30):
        loss = torch.nn.functional.cross_entropy(net(x), y)
        optimizer.zero_grad()
        loss.backward()
        optimizer.step()
        losses.append(float(loss))
    assert losses[-1] < 0.8 * losses[0]
