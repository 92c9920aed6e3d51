"""Kernels of the BitNet b1.58 layer against plain fp32 PyTorch expressions of the same functions.

A rounding kernel cannot agree bit for bit with an oracle that computes its scale in another
order: a value that lands within an ulp of a half flips to the neighbouring integer. The checks
therefore allow a small fraction of entries to differ, each by exactly one step."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    from ohara_b200.ops._ext import ext

    yield
    torch.cuda.synchronize()
    code, block, count, _ = ext().status(True)
    assert code == 0, f"kernel wait timed out: code={code} block={block} count={count}"


def _steps_apart(got, want, allowed_fraction):
    difference = (got.float() - want.float()).abs()
    assert float(difference.max()) <= 1.0, "an entry is off by more than one quantisation step"
    assert float((difference > 0).float().mean()) <= allowed_fraction


@pytest.mark.parametrize("rows,width", [(1, 8), (37, 264), (1000, 768), (4096, 2048)])
def test_activation_quantiser(rows, width):
    from ohara_b200.ops.bitnet import quantize_activations

    torch.manual_seed(rows)
    x = (torch.randn(rows, width, device="cuda") * 2.5).bfloat16()
    x[0] = 0                                            # a row of zeros takes the clamp
    q, dequant, rstd = quantize_activations(x)
    assert rstd is None and q.dtype == torch.bfloat16
    amax = x.float().abs().amax(dim=-1).clamp_min(1e-5)
    want = (x.float() * (127.0 / amax)[:, None]).round().clamp(-128, 127)
    _steps_apart(q, want, 1e-4)
    torch.testing.assert_close(dequant, amax / 127.0, rtol=1e-6, atol=0)

    weight = torch.empty(width, device="cuda").uniform_(0.5, 1.5)
    q, dequant, rstd = quantize_activations(x, weight, 1e-5)
    want_rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    normed = x.float() * want_rstd[:, None] * weight
    amax = normed.abs().amax(dim=-1).clamp_min(1e-5)
    want = (normed * (127.0 / amax)[:, None]).round().clamp(-128, 127)
    torch.testing.assert_close(rstd, want_rstd, rtol=1e-5, atol=0)
    torch.testing.assert_close(dequant, amax / 127.0, rtol=1e-5, atol=0)
    _steps_apart(q, want, 5e-3)


@pytest.mark.parametrize("shape,dtype", [((8, 8), torch.float32), ((768, 3072), torch.float32),
                                         ((1000, 520), torch.bfloat16), ((4096, 4096), torch.float32)])
def test_weight_quantiser(shape, dtype):
    from ohara_b200.ops.bitnet import quantize_weight

    torch.manual_seed(shape[0])
    w = (torch.randn(*shape, device="cuda") * 0.02).to(dtype)
    ternary, scale = quantize_weight(w)
    again, scale_again = quantize_weight(w)
    assert torch.equal(ternary, again) and torch.equal(scale, scale_again)   # fixed summation order
    mean = w.double().abs().mean().clamp_min(1e-5)
    torch.testing.assert_close(scale.double()[0], mean, rtol=1e-5, atol=0)
    want = (w.float() * (1.0 / mean.float())).round().clamp(-1, 1)
    assert ternary.dtype == torch.bfloat16 and ternary.shape == w.shape
    _steps_apart(ternary, want, 1e-4)


@pytest.mark.parametrize("rows,n_in,n_out,bias", [(256, 128, 128, False), (1024, 768, 512, True),
                                                  (2048, 768, 3072, False)])
def test_bit_linear_layer_forward_and_backward(rows, n_in, n_out, bias):
    from ohara_b200.ops.bitnet import bit_linear, bit_linear_reference

    torch.manual_seed(rows)
    x = torch.randn(rows, n_in, device="cuda").bfloat16().requires_grad_()
    weight = (torch.randn(n_out, n_in, device="cuda") * 0.05).requires_grad_()
    norm_weight = torch.empty(n_in, device="cuda").uniform_(0.5, 1.5).requires_grad_()
    b = torch.randn(n_out, device="cuda").requires_grad_() if bias else None
    grad = torch.randn(rows, n_out, device="cuda").bfloat16()
    inputs = [t for t in (x, weight, norm_weight, b) if t is not None]

    got = bit_linear(x, weight, norm_weight, b)
    got_grads = torch.autograd.grad(got, inputs, grad)
    x32 = x.detach().float().requires_grad_()
    reference_inputs = [x32] + inputs[1:]
    want = bit_linear_reference(x32, weight, norm_weight, b)
    want_grads = torch.autograd.grad(want, reference_inputs, grad.float())

    def close(have, ref, rtol, atol_rms, name):
        have, ref = have.float(), ref.float()
        atol = atol_rms * ref.square().mean().sqrt().item()
        excess = (have - ref).abs() - (atol + rtol * ref.abs())
        assert excess.max().item() <= 0, f"{name}: {int((excess > 0).sum())} of {ref.numel()} out"

    assert got.dtype == torch.bfloat16
    # a flipped activation moves one product term by one step of 1 / 127 of the row's maximum
    close(got, want, 1e-2, 2e-2, "output")
    for have, ref, name in zip(got_grads, want_grads, ("dx", "dweight", "dnorm", "dbias")):
        close(have, ref, 2e-2, 3e-2, name)
