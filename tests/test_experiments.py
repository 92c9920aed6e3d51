"""Contracts of the research modules under ``experiments/`` (CPU)."""

import torch
import torch.nn as nn

from experiments.bitnet.bitnet import BitLinear, activation_quant, apply_bitlinear, weight_quant
from experiments.deepseek_moe.dsmoe import DSMoE
from experiments.mhc.hyper_connections import HyperConnectedBlock, ManifoldHyperConnections
from experiments.misc.small_modules import (GaLoreProjector, Pattention, XLinear, relu_squared,
                                             silulu)
from experiments.mixture_of_depth.mod import MixtureOfDepth
from experiments.mla.mla import MLAConfig, MultiHeadLatentAttention
from experiments.q_sparse.q_sparse import QSparseLinear, q_sparse


def test_bitnet_quantisers_and_straight_through_gradients():
    torch.manual_seed(0)
    x = torch.randn(4, 16, requires_grad=True)
    y = activation_quant(x)
    levels = (y.detach() * 127.0 / x.detach().abs().amax(-1, keepdim=True))
    assert torch.allclose(levels, levels.round(), atol=1e-4) and levels.abs().max() <= 128
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))
    w = torch.randn(8, 16, requires_grad=True)
    wq, scale = weight_quant(w)
    assert set((wq.detach() * 1.0).round().unique().tolist()) <= {-1.0, 0.0, 1.0}
    (wq * scale).sum().backward()
    assert torch.allclose(w.grad, torch.ones_like(w))
    model = apply_bitlinear(nn.Sequential(nn.Linear(16, 32), nn.SiLU(), nn.Linear(32, 4)))
    assert all(isinstance(m, BitLinear) for m in model if isinstance(m, nn.Linear))
    model(torch.randn(3, 16)).sum().backward()
    assert all(p.grad is not None for p in model.parameters())


def test_q_sparse_keeps_top_k_and_passes_gradients_through():
    x = torch.tensor([[1.0, -3.0, 2.0, 0.5]], requires_grad=True)
    y = q_sparse(x, 2)
    assert y.tolist() == [[1.0, 0.0, 2.0, 0.0]]
    y.sum().backward()
    assert x.grad.tolist() == [[1.0, 1.0, 1.0, 1.0]]
    layer = QSparseLinear(0.5, 8, 4)
    assert layer.k == 4 and layer(torch.randn(2, 8)).shape == (2, 4)


def test_mla_is_causal_and_caches_a_small_latent():
    torch.manual_seed(0)
    cfg = MLAConfig(d_model=64, num_heads=4, v_head_dim=8, nope_head_dim=8, rope_head_dim=8,
                    q_lora_rank=16, kv_lora_rank=16, max_sequence_length=32)
    attn = MultiHeadLatentAttention(cfg).eval()
    x = torch.randn(2, 12, 64)
    full = attn(x)
    assert full.shape == (2, 12, 64)
    changed = x.clone()
    changed[:, 8:] += 1.0
    assert torch.allclose(attn(changed)[:, :8], full[:, :8], atol=1e-5)  # no look-ahead
    latent, rope_key = attn.latent_cache(x)
    assert latent.shape[-1] + rope_key.shape[-1] == 24 < 2 * 4 * 16


def test_dsmoe_bias_update_balances_load_without_an_auxiliary_loss():
    torch.manual_seed(0)
    moe = DSMoE(16, 32, num_experts=4, experts_per_token=2, num_shared_experts=1,
                expert_update_rate=0.05)
    with torch.no_grad():
        moe.gate.weight.normal_(std=0.3)
        moe.gate.weight[0] += 0.3  # inputs are positive: expert 0 is favoured at first
    x = torch.rand(4, 32, 16)
    moe.train()
    out, aux, first = moe(x)
    assert out.shape == x.shape and float(aux) == 0.0 and first > 0.0
    history = [moe(x)[2] for _ in range(60)]
    assert sum(history[-10:]) / 10 < 0.5 * first and moe.expert_biases[0] < 0
    moe.eval()
    before = moe.expert_biases.clone()
    moe(x)
    assert torch.equal(before, moe.expert_biases)
    with_loss = DSMoE(16, 32, num_experts=4, aux_free_loadbalancing=False, use_aux_loss=True)
    assert float(with_loss(x)[1]) > 0.0


def test_hyper_connections_produce_valid_mixing_objects():
    torch.manual_seed(0)
    hc = ManifoldHyperConnections(dim=8, rate=4, sinkhorn_iters=30)
    with torch.no_grad():
        hc.phi.normal_(std=0.5)
        hc.alpha.fill_(1.0)
    streams = torch.randn(2, 5, 4, 8)
    h_pre, h_post, h_res = hc(streams)
    assert h_pre.shape == (2, 5, 4) and (0 < h_pre).all() and (h_pre < 1).all()
    assert (0 < h_post).all() and (h_post < 2).all()
    assert torch.allclose(h_res.sum(-2), torch.ones(2, 5, 4), atol=1e-5)
    assert torch.allclose(h_res.sum(-1), torch.ones(2, 5, 4), atol=1e-2)
    block = HyperConnectedBlock(nn.Linear(8, 8), dim=8, rate=4)
    out = block(streams)
    assert out.shape == streams.shape
    out.sum().backward()
    assert block.connections.phi.grad is not None


def test_mixture_of_depth_touches_only_the_selected_tokens():
    torch.manual_seed(0)
    mod = MixtureOfDepth(nn.Linear(8, 8), dim=8, capacity_factor=0.25)
    x = torch.randn(2, 16, 8)
    out, loss = mod(x, auxiliary_loss=True)
    changed = (out != x).any(-1)
    assert changed.sum(1).tolist() == [4, 4]
    chosen = mod.router(x).squeeze(-1).topk(4, dim=1).indices
    assert all(changed[b, chosen[b]].all() for b in range(2))
    assert loss.item() > 0 and mod.select_for_decoding(x).shape == (2, 16)


def test_small_modules():
    x = torch.randn(5, 6, requires_grad=True)
    y = relu_squared(x)
    y.sum().backward()
    assert torch.allclose(y, torch.relu(x).square())
    assert torch.allclose(x.grad, 2 * torch.relu(x.detach()))
    assert torch.allclose(silulu(x), torch.nn.functional.silu(x) + torch.relu(x).square())
    plain, xl = nn.Linear(6, 3), XLinear(6, 3)
    xl.load_state_dict(plain.state_dict())
    assert torch.allclose(xl(x), plain(x), atol=1e-5)  # same function, different parametrisation
    pat = Pattention(6, 4, num_tokens=10)
    before = pat(x)
    pat.expand_tokens(14)
    assert pat.keys.shape == (14, 6) and pat(x).shape == before.shape
    grad = torch.randn(12, 3) @ torch.randn(3, 20)  # rank 3
    proj = GaLoreProjector(rank=3)
    low = proj.project(grad, step=0)
    assert low.shape == (3, 20)
    assert torch.allclose(proj.project_back(low), grad, atol=1e-4)
    tall = GaLoreProjector(rank=3)
    assert tall.project(grad.t().contiguous(), 0).shape == (20, 3)
