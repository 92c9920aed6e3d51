"""Run-to-run determinism as a cheap race detector (no memory checker is available on the device).

Every kernel whose algorithm fixes the order of its floating-point operations must return the same
bits when it is run again on the same inputs, also when the memory its outputs and scratch buffers
land in was filled with NaN bit patterns beforehand (a kernel that leaves part of its output
unwritten, or reads a staging buffer before it is filled, shows up as a difference). Kernels that
accumulate with floating-point atomics (dQ of attention, split-K weight gradients) are only
required to be finite and close.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(*shape):
    return torch.randn(*shape, device="cuda").bfloat16()


def poison(*sizes_bytes):
    """Fill freshly freed allocator blocks of the given sizes with NaN patterns: the next
    ``torch.empty`` of such a size is served from them."""
    blocks = [torch.full((max(size // 4, 1),), float("nan"), device="cuda") for size in sizes_bytes]
    torch.cuda.synchronize()
    del blocks


def run_twice(fn, output_bytes):
    first = [t.clone() for t in fn()]
    torch.cuda.synchronize()
    poison(*output_bytes)
    second = fn()
    torch.cuda.synchronize()
    return first, list(second)


def assert_same_bits(first, second, names):
    for a, b, name in zip(first, second, names):
        assert not torch.isnan(b.float()).any(), f"{name}: NaN (unwritten output)"
        assert torch.equal(a, b), f"{name}: differs between two runs"


@pytest.fixture(autouse=True)
def _status_clean():
    from ohara_b200.ops._ext import ext

    yield
    torch.cuda.synchronize()
    code, block, count, _ = ext().status(True)
    assert code == 0, f"kernel wait timed out: code={code} block={block} count={count}"


@pytest.mark.parametrize("m,n,k", [(1000, 768, 520), (4096, 2048, 768), (130, 96, 64)])
def test_gemm_nt_and_nn_are_bitwise_reproducible(m, n, k):
    from ohara_b200 import ops

    torch.manual_seed(0)
    a, w = bf(m, k), bf(n, k)
    first, second = run_twice(lambda: (ops.matmul_nt(a, w), ops.matmul_nn(ops.matmul_nt(a, w), w)),
                              [m * n * 2, m * k * 2])
    assert_same_bits(first, second, ["nt", "nn"])


def test_attention_forward_and_key_value_gradients_are_bitwise_reproducible():
    from ohara_b200.ops.attention import attention

    torch.manual_seed(0)
    q, k, v = bf(2, 700, 4, 128), bf(2, 700, 2, 128), bf(2, 700, 2, 128)
    upstream = bf(2, 700, 4, 128)

    def step():
        qs, ks, vs = (t.detach().requires_grad_() for t in (q, k, v))
        out = attention(qs, ks, vs, causal=True)
        out.backward(upstream)
        return out.detach(), ks.grad, vs.grad, qs.grad

    first, second = run_twice(step, [q.numel() * 2, k.numel() * 2, k.numel() * 2, q.numel() * 4])
    assert_same_bits(first[:3], second[:3], ["out", "dk", "dv"])
    # dQ is accumulated with floating-point atomics: order-dependent in the last bits only
    assert torch.isfinite(second[3].float()).all()
    scale = first[3].float().abs().max().item()
    assert (first[3].float() - second[3].float()).abs().max().item() <= 2e-2 * scale


def test_normalisation_activation_and_rope_are_bitwise_reproducible():
    from ohara_b200 import ops

    torch.manual_seed(0)
    x, delta = bf(777, 768), bf(777, 768)
    weight = 1 + 0.1 * torch.randn(768, device="cuda")
    gate, up = bf(777, 512), bf(777, 512)
    q, k = bf(2, 300, 4, 128), bf(2, 300, 2, 128)
    angles = torch.outer(torch.arange(300, device="cuda").float(),
                         1.0 / 10000 ** (torch.arange(0, 128, 2, device="cuda").float() / 128))
    cos, sin = angles.cos(), angles.sin()

    def step():
        xs, ds, ws = x.detach().requires_grad_(), delta.detach().requires_grad_(), weight.detach().requires_grad_()
        y, s = ops.add_rms_norm(xs, ds, ws, 1e-5)
        gs, us = gate.detach().requires_grad_(), up.detach().requires_grad_()
        act = ops.swiglu(gs, us)
        torch.autograd.backward([y, s, act], [x, delta, gate])
        qo, ko = ops.rope_qk(q, k, cos, sin)
        return y.detach(), s.detach(), xs.grad, ds.grad, act.detach(), gs.grad, us.grad, qo, ko

    first, second = run_twice(step, [x.numel() * 2] * 4 + [gate.numel() * 2] * 3 + [q.numel() * 2, k.numel() * 2])
    assert_same_bits(first, second, ["y", "sum", "dx", "ddelta", "swiglu", "dgate", "dup", "q", "k"])


def test_fused_loss_is_bitwise_reproducible():
    from ohara_b200 import ops

    torch.manual_seed(0)
    hidden, weight = bf(1500, 256), torch.randn(1000, 256, device="cuda") * 0.05
    targets = torch.randint(0, 1000, (1500,), device="cuda")
    targets[::7] = -1

    def step():
        hs = hidden.detach().requires_grad_()
        loss = ops.linear_cross_entropy(hs, weight, targets, -1, 1.0 / 1500)
        loss.backward()
        return loss.detach().reshape(1), hs.grad

    first, second = run_twice(step, [hidden.numel() * 2, 1500 * 1000 * 2])
    assert_same_bits(first, second, ["loss", "dhidden"])


def test_moe_dispatch_experts_and_combine_are_bitwise_reproducible():
    from ohara_b200.modules.moe_grouped import GroupedMoE
    from ohara_b200.ops.grouped import grouped_swiglu_experts

    torch.manual_seed(0)
    moe = GroupedMoE(dim=128, hidden_dim=64, num_experts=8, num_experts_per_tok=2,
                     num_shared_experts=0, gate_fn="sigmoid").cuda()
    with torch.no_grad():
        moe.w_down.normal_(std=0.05)
    flat = bf(900, 128)
    indices, weights, _, _ = moe._route(flat)

    def step():
        xs = flat.detach().requires_grad_()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = grouped_swiglu_experts(xs, indices, weights.detach(), moe.w_gate, moe.w_up, moe.w_down)
        out.backward(flat)
        return out.detach(), xs.grad

    first, second = run_twice(step, [flat.numel() * 2, (900 * 2 + 8 * 256) * 128 * 2,
                                     (900 * 2 + 8 * 256) * 64 * 2])
    assert_same_bits(first, second, ["moe_out", "dx"])


def test_scan_kernels_are_bitwise_reproducible():
    from ohara_b200.modules.pscan import pscan

    torch.manual_seed(0)
    a = torch.rand(2, 257, 96, device="cuda") * 0.5 + 0.5
    x = torch.randn(2, 257, 96, device="cuda")

    def step():
        as_, xs = a.detach().requires_grad_(), x.detach().requires_grad_()
        h = pscan(as_, xs)
        h.backward(x)
        return h.detach(), as_.grad, xs.grad

    first, second = run_twice(step, [a.numel() * 4] * 3)
    assert_same_bits(first, second, ["h", "da", "dx"])
