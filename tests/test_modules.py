"""Building blocks: KV cache, rotary/ALiBi/XPos, attention, MLPs, MoE + balancing, scans, adapters
and small utilities. Behaviour follows the reference suite (tests/test_modules.py:46-353)."""

from __future__ import annotations

import math
import re

import pytest
import torch
import torch.nn as nn

from ohara_b200.adaptor.dora import DoRALinear, merge_dora, replace_with_dora
from ohara_b200.adaptor.lora import LoRALinear, mark_lora_as_trainable, merge_lora, replace_with_lora
from ohara_b200.embeddings_pos.alibi import get_alibi_mask
from ohara_b200.embeddings_pos.rotary import RoPE, apply_rope, precompute_freqs_cis
from ohara_b200.embeddings_pos.xpos import XPos
from ohara_b200.modules.attention import Attention, CasualAttention, CausalAttention
from ohara_b200.modules.kv_cache import KVCache, dequantize_int8, quantize_int8
from ohara_b200.modules.linear_rnn import Hawk, RG_LRU
from ohara_b200.modules.mlp import MLP_MAP
from ohara_b200.modules.moe import MoE, apply_qb_update, expert_load, maximal_violation
from ohara_b200.modules.norm import RMSNorm
from ohara_b200.modules.pscan import pscan, sequential_scan
from ohara_b200.swa import make_swa_mask, sliding_window_attention_with_mask
from ohara_b200.utils import BetterCycle, build_mask, random_name


# -- KV cache --------------------------------------------------------------------------------------
def test_cache_returns_everything_written_and_enforces_order():
    cache = KVCache((2, 8, 2, 4), max_seq_length=8, dtype=torch.float32)
    first, second = torch.randn(2, 3, 2, 4), torch.randn(2, 1, 2, 4)
    keys, values = cache.forward(first, first * 2, 0)
    assert keys.shape == (2, 3, 2, 4) and torch.equal(values, first * 2)
    keys, _ = cache.forward(second, second, 3)
    assert torch.equal(keys, torch.cat([first, second], dim=1))
    with pytest.raises(ValueError, match="sequential"):
        cache.forward(second, second, 7)
    with pytest.raises(ValueError, match="matching shapes"):
        cache.forward(second, second[:, :, :1], 4)
    with pytest.raises(ValueError, match="batch size cannot change"):
        cache.forward(second[:1], second[:1], 4)
    with pytest.raises(ValueError, match="exceeds"):
        cache.forward(torch.randn(2, 5, 2, 4), torch.randn(2, 5, 2, 4), 4)
    cache.reset()
    assert cache.forward(second[:1], second[:1], 0)[0].shape == (1, 1, 2, 4)


def test_int8_cache_is_close_to_the_original():
    x = torch.randn(3, 5, 2, 16)
    q, scale, low = quantize_int8(x)
    assert q.dtype == torch.int8
    assert (dequantize_int8(q, scale, low) - x).abs().max() <= scale.max() * 0.51
    cache = KVCache((3, 8, 2, 16), max_seq_length=8, dtype=torch.float32, int8=True)
    keys, values = cache.forward(x, -x, 0)
    assert keys.dtype == torch.float32 and torch.allclose(keys, x, atol=0.03)
    assert torch.allclose(values, -x, atol=0.03)


# -- positions ---------------------------------------------------------------------------------------
def test_rope_is_a_rotation():
    q, k = torch.randn(2, 6, 3, 8), torch.randn(2, 6, 3, 8)
    cos, sin = precompute_freqs_cis(8, 6)
    rq, rk = apply_rope(q, k, (cos, sin))
    assert rq.shape == q.shape
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    assert torch.allclose(rq[:, 0], q[:, 0], atol=1e-6), "position 0 is not rotated"
    # relative property: <R_m q, R_n k> depends only on m - n
    same_q, same_k = q[:, :1].expand(-1, 6, -1, -1), k[:, :1].expand(-1, 6, -1, -1)
    a, b = apply_rope(same_q, same_k, (cos, sin))
    dots = torch.einsum("bthd,bshd->bhts", a, b)
    assert torch.allclose(dots[..., 1, 0], dots[..., 4, 3], atol=1e-4)


def test_rope_module_rotates_only_the_leading_dims():
    x = torch.randn(2, 5, 12)
    y = RoPE(8)(x)
    assert y.shape == x.shape and torch.equal(y[..., 8:], x[..., 8:])
    assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1), atol=1e-5)
    full = RoPE(12, traditional=True)(x)
    assert torch.allclose(full.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    with pytest.raises(NotImplementedError):
        RoPE(8, traditional=True)(x)
    shifted = RoPE(8)(x[:, 2:], offset=2)
    assert torch.allclose(shifted, RoPE(8)(x)[:, 2:], atol=1e-6)
    with pytest.raises(ValueError):
        RoPE(7)


def test_alibi_and_xpos_masks():
    mask = get_alibi_mask(4, 6)
    assert mask.shape == (4, 6, 6)
    row = mask[0, 5]
    assert all(row[i] < row[i + 1] < 0 for i in range(5)), "older keys are penalised more"
    assert torch.all(mask.triu(1) == 0), "future keys carry no penalty (the causal mask hides them)"
    assert mask[3, 5, 0] > mask[0, 5, 0], "later heads decay slower"
    (cos, sin), decay = XPos(dim=32, num_heads=4)(5)
    assert cos.shape == sin.shape == (5, 8) and decay.shape == (4, 5, 5)
    assert torch.all(decay.triu(1) == 0) and torch.all(decay.diagonal(dim1=1, dim2=2) > 0)
    _, scalar = XPos(dim=32, num_heads=4)(5, recurrent=True)
    assert scalar.shape == (4,) and torch.all((scalar > 0) & (scalar < 1))


def test_masks():
    causal = build_mask(4)
    assert causal.shape == (1, 1, 4, 4)
    assert torch.equal(causal[0, 0] == 0, torch.ones(4, 4).tril().bool())
    window = build_mask(5, sliding_window_attention=True, window_size=2)[0, 0] == 0
    assert window[4].tolist() == [False, False, False, True, True]
    keep = make_swa_mask(6, 3, device=torch.device("cpu"), dtype=torch.float32)
    q, k, v = (torch.randn(2, 6, 4) for _ in range(3))  # (B, T, D), unscaled scores
    out = sliding_window_attention_with_mask(q, k, v, window_size=3)
    scores = q @ k.transpose(-1, -2)
    visible = torch.tensor([[0 <= i - j < 3 for j in range(6)] for i in range(6)])
    manual = torch.softmax(scores.masked_fill(~visible, float("-inf")), dim=-1) @ v
    assert torch.allclose(out, manual, atol=1e-5)
    assert keep.shape[-2:] == (6, 6)


# -- attention / norm / MLP ----------------------------------------------------------------------------
def test_causal_attention_is_causal():
    assert Attention is CausalAttention and CasualAttention is CausalAttention
    attn = CausalAttention(16, 4).eval()
    x = torch.randn(2, 5, 16)
    out, info = attn(x, verbose=True)
    assert out.shape == x.shape and info["attn_mtx"].shape == (2, 4, 5, 5)
    assert torch.all(info["attn_mtx"].triu(1) == 0)
    assert torch.allclose(info["attn_mtx"].sum(-1), torch.ones(2, 4, 5), atol=1e-5)
    assert torch.allclose(attn(x), out, atol=1e-5), "fused and explicit paths agree"
    changed = x.clone()
    changed[:, -1] += 1.0
    assert torch.allclose(attn(changed)[:, :-1], out[:, :-1], atol=1e-6)
    with pytest.raises(ValueError):
        CausalAttention(10, 4)


def test_rmsnorm_gives_unit_rms():
    y = RMSNorm(32)(torch.randn(4, 32) * 7)
    assert torch.allclose(y.pow(2).mean(-1).sqrt(), torch.ones(4), atol=1e-3)


@pytest.mark.parametrize("name", sorted(MLP_MAP))
def test_mlp_variants_keep_the_shape_and_train(name):
    block = MLP_MAP[name](16, 32)
    x = torch.randn(2, 3, 16, requires_grad=True)
    y = block(x)
    assert y.shape == x.shape
    y.sum().backward()
    assert x.grad is not None and all(p.grad is not None for p in block.parameters())


# -- mixture of experts ------------------------------------------------------------------------------
def test_moe_equals_a_per_token_loop_and_trains_what_it_used():
    torch.manual_seed(0)
    moe = MoE(8, 16, num_experts=4, num_experts_per_tok=2, quantile_balancing=False)
    x = torch.randn(2, 5, 8)
    out = moe(x)
    flat = x.reshape(-1, 8)
    scores = flat @ moe.gate.weight.t()
    expected = torch.zeros_like(flat)
    for t in range(flat.size(0)):
        top = scores[t].topk(2)
        for weight, index in zip(top.values.softmax(-1), top.indices):
            expected[t] += weight * moe.experts[int(index)](flat[t : t + 1])[0]
    assert torch.allclose(out.reshape(-1, 8), expected, atol=1e-5)
    out.sum().backward()
    used = set(scores.topk(2).indices.flatten().tolist())
    assert moe.gate.weight.grad.abs().sum() > 0
    for index, expert in enumerate(moe.experts):
        touched = any(p.grad is not None and p.grad.abs().sum() > 0 for p in expert.parameters())
        assert touched == (index in used)


def test_quantile_balancing_levels_the_load():
    torch.manual_seed(1)
    with pytest.raises(AssertionError, match="threshold"):
        MoE(8, 16, num_experts=2, num_experts_per_tok=2)
    moe = MoE(8, 16, num_experts=8, num_experts_per_tok=2).train()
    with torch.no_grad():
        moe.gate.weight[0] += 2.0  # a router that loves expert 0
        moe.gate.weight[0].abs_()
    x = torch.randn(4, 64, 8).abs()
    moe(x)
    assert torch.all(moe.router_bias == 0), "nothing moves until the update is applied"
    before = maximal_violation(moe.expert_load())
    for _ in range(30):
        moe(x)
        apply_qb_update(moe)
    moe.expert_load()
    moe(x)
    counts = expert_load(moe)[0]
    assert int(counts.sum()) == 4 * 64 * 2
    assert maximal_violation(counts) < 0.5 * before
    assert abs(float(moe.router_bias.mean())) < 1e-6
    assert int(moe.expert_counts.sum()) == 0, "reading the load resets it"
    moe.eval()
    moe(x)
    assert int(moe.expert_counts.sum()) == 0


# -- scans and recurrent blocks ---------------------------------------------------------------------
def test_parallel_scan_matches_the_recurrence_with_gradients():
    a = torch.rand(2, 16, 3, 4, dtype=torch.float64, requires_grad=True)
    x = torch.randn(2, 16, 3, 4, dtype=torch.float64, requires_grad=True)
    fast, slow = pscan(a, x), sequential_scan(a, x)
    assert torch.allclose(fast, slow, atol=1e-10)
    grads_fast = torch.autograd.grad(fast.square().sum(), (a, x))
    grads_slow = torch.autograd.grad(slow.square().sum(), (a, x))
    for g_fast, g_slow in zip(grads_fast, grads_slow):
        assert torch.allclose(g_fast, g_slow, atol=1e-9)


@pytest.mark.parametrize("shape", [(2, 7, 5), (3, 33, 300), (2, 64, 40, 30), (1, 1, 3), (2, 5, 1100)])
def test_host_scan_kernel_matches_the_recurrence_with_gradients(shape):
    """fp32 CPU tensors run the one-pass kernel of the extension (when it is built); whole and
    partial channel blocks, one step, non-contiguous inputs."""
    from ohara_b200.modules.pscan import PScan, _native_cpu_scan

    if not _native_cpu_scan():
        pytest.skip("the extension is not built")
    torch.manual_seed(0)
    a = torch.rand(shape).transpose(0, 1).contiguous().transpose(0, 1).requires_grad_()
    x = torch.randn(shape, requires_grad=True)
    upstream = torch.randn(shape)
    got = pscan(a, x)
    got_grads = torch.autograd.grad(got, (a, x), upstream)
    a64, x64 = a.detach().double().requires_grad_(), x.detach().double().requires_grad_()
    want = sequential_scan(a64, x64)
    want_grads = torch.autograd.grad(want, (a64, x64), upstream.double())
    torch.testing.assert_close(got.double(), want, rtol=1e-5, atol=1e-5)
    for have, ref in zip(got_grads, want_grads):
        torch.testing.assert_close(have.double(), ref, rtol=1e-5, atol=1e-5)
    doubling = PScan.apply(a.detach(), x.detach())          # the PyTorch form agrees as well
    torch.testing.assert_close(doubling, got.detach(), rtol=1e-5, atol=1e-5)
    threads = torch.get_num_threads()
    torch.set_num_threads(1)                                  # one thread: the serial path
    try:
        with torch.no_grad():
            torch.testing.assert_close(pscan(a, x), got.detach(), rtol=0, atol=0)
    finally:
        torch.set_num_threads(threads)


def test_recurrent_blocks_are_causal():
    for block in (RG_LRU(16), Hawk(dim=16)):
        block.eval()
        x = torch.randn(2, 9, 16)
        base = block(x)
        assert base.shape == x.shape
        x2 = x.clone()
        x2[:, -1] += 1
        assert torch.allclose(block(x2)[:, :-1], base[:, :-1], atol=1e-5)
        x3 = x.clone()
        x3[:, 2] += 1
        later = (block(x3) - base)[:, 3:].abs().amax(dim=(0, 2))
        assert (later > 1e-4).all()          # and it has a memory: later steps see the change


# -- adapters ----------------------------------------------------------------------------------------
class Nest(nn.Module):
    def __init__(self):
        super().__init__()
        self.first = nn.Linear(8, 8)
        self.inner = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))

    def forward(self, x):
        return self.inner(self.first(x))


@pytest.mark.parametrize("replace, merge, kind", [(replace_with_lora, merge_lora, LoRALinear),
                                                  (replace_with_dora, merge_dora, DoRALinear)])
def test_adapters_replace_train_and_merge(replace, merge, kind):
    torch.manual_seed(0)
    model, x = Nest(), torch.randn(3, 8)
    before = model(x)
    replace(model, rank=2)
    wrapped = [m for m in model.modules() if isinstance(m, kind)]
    assert len(wrapped) == 3
    assert torch.allclose(model(x), before, atol=1e-5), "a fresh adapter is the identity"
    if kind is LoRALinear:
        mark_lora_as_trainable(model)
        trainable = {n for n, p in model.named_parameters() if p.requires_grad}
        assert trainable and all("lora" in n for n in trainable)
    for module in wrapped:
        for p in module._adapter_parameters():
            nn.init.normal_(p, std=0.1) if p.dim() > 1 else None
    adapted = model(x)
    assert not torch.allclose(adapted, before, atol=1e-4)
    merge(model)
    assert torch.allclose(model(x), adapted, atol=1e-4)


# -- utilities -----------------------------------------------------------------------------------------
def test_cycle_and_run_names():
    cycle = BetterCycle([1, 2, 3])
    assert [next(cycle) for _ in range(7)] == [1, 2, 3, 1, 2, 3, 1] and cycle.idx == 2
    cycle.close()
    assert cycle._iterator is None and next(cycle) == 1
    assert re.fullmatch(r"[a-z0-9_\-]+-\d{4}(_\d{2}){5}", random_name(), flags=re.I)


def test_small_helpers_of_the_public_surface():
    """Names the reference exports that nothing else here needs: rotary table broadcasting,
    power-of-two padding for scans, the model holder of the summary utility, the name pool."""
    import torch

    from ohara_b200.embeddings_pos.rotary import precompute_freqs_cis, reshape_for_broadcast
    from ohara_b200.modules.pscan import npo2, pad_npo2
    from ohara_b200.utils.info import Model, model_summary
    from ohara_b200.utils.rand import pokemon_names, random_name

    cos, _ = precompute_freqs_cis(8, 6)
    x = torch.zeros(2, 6, 3, 4)
    assert reshape_for_broadcast(cos, x).shape == (1, 6, 1, 4)
    with pytest.raises(ValueError):
        reshape_for_broadcast(cos, torch.zeros(2, 5, 3, 4))
    assert [npo2(n) for n in (1, 2, 3, 8, 9, 1000)] == [1, 2, 4, 8, 16, 1024]
    padded = pad_npo2(torch.ones(2, 5, 3, 1))
    assert padded.shape == (2, 8, 3, 1) and float(padded[:, 5:].abs().sum()) == 0
    assert pad_npo2(torch.ones(1, 4, 2, 2)).shape == (1, 4, 2, 2)
    holder = Model(torch.nn.Linear(3, 2))
    assert holder(torch.zeros(1, 3)).shape == (1, 2)
    assert model_summary(holder)["total_parameters"] == "8"
    names = pokemon_names()
    assert len(names) > 10 and random_name().split("-")[0] in names
