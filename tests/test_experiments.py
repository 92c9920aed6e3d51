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
        for phi in (hc.phi_pre, hc.phi_post, hc.phi_res):
            phi.normal_(std=0.5)
        for alpha in (hc.alpha_pre, hc.alpha_post, hc.alpha_res):
            alpha.fill_(1.0)
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
    assert block.connections.phi_res.grad is not None


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
    unit = plain.weight / plain.weight.norm(dim=-1, keepdim=True)
    assert torch.allclose(xl(x), torch.nn.functional.linear(x, unit, plain.bias), atol=1e-6)
    with torch.no_grad():
        xl.weight.mul_(3.0)                       # only the direction of a row matters
    assert torch.allclose(xl(x), torch.nn.functional.linear(x, unit, plain.bias), atol=1e-5)
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


# --------------------------------------------------------------------------------------------------
# Recurrent models, attention variants, feed-forward variants, data, optimizers
# --------------------------------------------------------------------------------------------------
def test_griffin_hawk_and_mqa_models_train_and_the_recurrence_steps_like_the_scan():
    import pytest
    from experiments.griffin_and_hawk.model import (HawkAndGriffin, HawkState, HnGConfig, hawk_step,
                                                    state_floats_per_sequence)
    from ohara_b200.modules.linear_rnn import Hawk

    torch.manual_seed(0)
    tokens = torch.randint(0, 50, (2, 16))
    for kind in ("mqa", "hawk", "griffin"):
        cfg = HnGConfig(model_type=kind, vocab_size=50, seq_len=32, dim=32, num_heads=4,
                        num_kv_heads=1, num_layers=2, sliding_window_attention=kind == "griffin",
                        window_size=4)
        model = HawkAndGriffin(cfg)
        logits = model(tokens)
        assert logits.shape == (2, 16, 50)
        changed = tokens.clone()
        changed[:, 10:] = (changed[:, 10:] + 1) % 50
        assert torch.allclose(model(changed)[:, :10], logits[:, :10], atol=1e-5)  # causal
        torch.nn.functional.cross_entropy(logits.flatten(0, 1), tokens.flatten()).backward()
        assert all(p.grad is not None for p in model.parameters())
        sizes = state_floats_per_sequence(cfg, 4096)
        assert (sizes["recurrent_state"] > 0) == (kind != "mqa")
        assert (sizes["kv_cache"] > 0) == (kind != "hawk")
    with pytest.raises(ValueError):
        HawkAndGriffin(HnGConfig(model_type="owl", vocab_size=8, dim=16, num_heads=2, num_layers=1))
    # a window of 4 hides position 0 from position 8
    local = HawkAndGriffin(HnGConfig(model_type="mqa", vocab_size=50, seq_len=32, dim=32,
                                     num_heads=4, num_layers=1, sliding_window_attention=True,
                                     window_size=4)).eval()
    far = tokens.clone()
    far[:, 0] = (far[:, 0] + 1) % 50
    assert torch.allclose(local(far)[:, 8:], local(tokens)[:, 8:], atol=1e-5)
    mixer = Hawk(dim=16, expansion_factor=1.5, kernel_size=4)
    x = torch.randn(2, 9, 16)
    state, outs = HawkState.zeros(mixer, 2), []
    for t in range(9):
        out, state = hawk_step(mixer, x[:, t], state)
        outs.append(out)
    assert torch.allclose(torch.stack(outs, 1), mixer(x), atol=1e-5)


def test_partial_kv_attention_variants_are_causal_and_cache_less():
    from experiments.partial_kv.pkv import ATTENTION, PartialKVAttention, cache_floats_per_token
    from ohara_b200.embeddings_pos.rotary import precompute_freqs_cis

    torch.manual_seed(0)
    x = torch.randn(2, 10, 32)
    later = x.clone()
    later[:, 6:] += 1.0
    for kind, cls in ATTENTION.items():
        layer = cls(32, 4).eval()
        cos, sin = precompute_freqs_cis(4 if kind == "partial_kv" else 8, 32)
        freqs = (cos[:10], sin[:10])
        out = layer(x, freqs)
        assert out.shape == x.shape
        assert torch.allclose(layer(later, freqs)[:, :6], out[:, :6], atol=1e-5)
    sizes = {kind: cache_floats_per_token(kind, 32, 2) for kind in ATTENTION}
    assert sizes == {"attention": 128, "kattention": 64, "partial_kv": 96}
    layer = PartialKVAttention(32, 4)
    cos, sin = precompute_freqs_cis(4, 32)
    key, shared, value = layer.cached(x, (cos[:10], sin[:10]))
    assert key.shape == shared.shape == value.shape == (2, 10, 4, 4)


def test_xglu_springnet_deglu_and_the_state_shift_loss():
    from experiments.deglu.deglu import DeGLU
    from experiments.mihawk.state_shift import state_prediction_loss, states_shift
    from experiments.springnet.springnet import SpringMLP
    from experiments.xglu.xglu import XGLU

    torch.manual_seed(0)
    x = torch.randn(2, 6, 32)
    layer = XGLU(32, xglu_rank=8)
    assert layer(x).shape == x.shape and layer.parameter_saving() > 0
    layer(x).sum().backward()
    assert layer.compress.weight.grad.abs().sum() > 0
    spring = SpringMLP(32, 48, spring_steps=5)
    out, step = spring(x)
    assert out.shape == x.shape and step.shape == (2, 6, 1)
    sizes = spring.step_sizes(x)
    assert bool((sizes[1:] <= sizes[:-1]).all()) and float(sizes.max()) < 1.0   # a damped motion
    (out.square().mean() + step.mean()).backward()
    assert spring.decay[0].weight.grad is not None
    deglu = DeGLU(32, 64, mask_blocks=4)
    hidden = torch.randn(5, 64)
    mask = deglu.get_mask(hidden)
    assert set(mask.unique().tolist()) <= {0.0, 1.0} and float(mask.sum()) % 16 == 0
    assert float(mask.sum()) >= 16 and deglu(x).shape == x.shape
    states = torch.arange(10.0).view(1, 10, 1)
    assert states_shift(states, 2)[0, :, 0].tolist() == [2, 3, 4, 5, 6, 7, 8, 9, 0, 0]
    assert states_shift(states, 0) is states
    # every state is 2 below its successor two steps on; 8 of 10 positions count
    assert abs(float(state_prediction_loss(states, 2)) - 4.0 * 8 / 10) < 1e-6


def test_game_of_life_rule_dataset_and_token_layout():
    from experiments.lifelm.life import (SEP, LifeDataset, boards_to_tokens, next_state,
                                         next_state_loops)

    torch.manual_seed(0)
    boards = (torch.rand(3, 7, 9) < 0.4).long()
    stepped = next_state(boards)
    for b in range(3):
        assert torch.equal(stepped[b], next_state_loops(boards[b]))
    blinker = torch.zeros(5, 5, dtype=torch.long)
    blinker[2, 1:4] = 1
    assert torch.equal(next_state(next_state(blinker)), blinker)
    assert not torch.equal(next_state(blinker), blinker)
    pairs = list(LifeDataset(size=6, samples=40, seed=1))
    assert len(pairs) == 40
    assert all(torch.equal(next_state(a), b) for a, b in pairs)
    tokens, mask = boards_to_tokens(*pairs[0])
    assert tokens.shape == (73,) and int(tokens[36]) == SEP and int(mask.sum()) == 36
    assert not bool(mask[:37].any())


def test_dense_mlp_decomposes_into_experts_that_sum_to_it():
    from experiments.mlp_decomp_to_moe.make_moe import (balanced_kmeans, decompose_gated_mlp,
                                                        split_weights_into_experts)
    from ohara_b200.modules.mlp import SwiGLU

    torch.manual_seed(0)
    points = torch.cat([torch.randn(40, 8) + 6 * torch.eye(8)[i] for i in range(4)])
    labels = balanced_kmeans(points, 4)
    assert torch.bincount(labels).tolist() == [40] * 4
    # well separated blobs are recovered
    assert all(len(set(labels[i * 40:(i + 1) * 40].tolist())) == 1 for i in range(4))
    parts = split_weights_into_experts(torch.randn(64, 16), 8)
    assert [p.shape for p in parts] == [(8, 16)] * 8
    mlp = SwiGLU(16, 64)
    x = torch.randn(3, 5, 16)
    everything = decompose_gated_mlp(mlp, num_experts=8, top_k=8)
    assert torch.allclose(everything(x), mlp(x), atol=1e-5)
    some = decompose_gated_mlp(mlp, num_experts=8, top_k=2)
    assert some(x).shape == x.shape and not torch.allclose(some(x), mlp(x), atol=1e-5)


def test_galore_adamw_keeps_low_rank_moments_and_trains():
    from experiments.galore.galore import GaLoreAdamW, galore_param_groups

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(24, 32), nn.Tanh(), nn.Linear(32, 24))
    optimizer = GaLoreAdamW(galore_param_groups(model, rank=4, update_proj_gap=5), lr=3e-2)
    x = torch.randn(64, 24)
    losses = []
    for _ in range(30):
        loss = (model(x) - x).square().mean()
        optimizer.zero_grad()
        loss.backward()
        optimizer.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < 0.7 * losses[0]
    assert optimizer.state[model[0].weight]["exp_avg"].shape == (32, 4)   # out >= in: (out, rank)
    assert optimizer.state[model[2].weight]["exp_avg"].shape == (4, 32)   # out < in: (rank, in)
    full = 2 * sum(p.numel() for p in model.parameters())
    assert optimizer.state_numbers() < 0.5 * full


def test_monkey_patcher_swaps_linears_and_keeps_the_function():
    from experiments.template.monkey_patcher import DMLinear, patch_linears

    torch.manual_seed(0)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.up, self.down = nn.Linear(8, 16), nn.Linear(16, 8, bias=False)
            self.inner = nn.Sequential(nn.Linear(8, 8))

        def forward(self, x):
            return self.inner(self.down(torch.relu(self.up(x))))

    net, x = Net(), torch.randn(4, 8)
    before = net(x)
    assert patch_linears(net, {"up", "down"}) == ["up", "down"]
    assert isinstance(net.up, DMLinear) and isinstance(net.inner[0], nn.Linear)
    assert not isinstance(net.inner[0], DMLinear)
    assert torch.allclose(net(x), before, atol=1e-5)
    assert patch_linears(net) == ["inner.0"]
    assert torch.allclose(net(x), before, atol=1e-5)


def test_bitlora_starts_as_the_base_layer_trains_only_adapters_and_merges():
    from experiments.bitnet.bitlora import BitLora, apply_bitlora

    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 6))
    x = torch.randn(5, 8)
    base = apply_bitlinear(nn.Sequential(*[m if not isinstance(m, nn.Linear) else
                                            _clone_linear(m) for m in net]))(x)
    apply_bitlora(net, rank=2, lora_alpha=4.0)
    assert all(isinstance(m, BitLora) for m in net if isinstance(m, nn.Linear))
    assert torch.allclose(net(x), base, atol=1e-6)             # B = 0: nothing changes yet
    trainable = {n for n, p in net.named_parameters() if p.requires_grad}
    assert trainable == {"0.lora_A", "0.lora_B", "2.lora_A", "2.lora_B"}
    net(x).square().mean().backward()
    assert net[0].lora_B.grad.abs().sum() > 0 and net[0].weight.grad is None
    with torch.no_grad():
        net[0].lora_B.normal_()
    adapted = net(x)
    net[0].merge()
    assert net[0].merged and torch.allclose(net(x), adapted, atol=1e-5)


def _clone_linear(linear: nn.Linear) -> nn.Linear:
    copy = nn.Linear(linear.in_features, linear.out_features, linear.bias is not None)
    copy.load_state_dict(linear.state_dict())
    return copy


def test_connection_types_of_the_mhc_model_and_template_variants_run_and_learn():
    from experiments.mhc.model import MHCConfig, MHCModel
    from experiments.template.model import VARIANTS, TemplateConfig, build
    from experiments.train_experiment import main

    torch.manual_seed(0)
    tokens = torch.randint(0, 40, (2, 12))
    for kind in ("residual", "hc", "mhc"):
        model = MHCModel(MHCConfig(vocab_size=40, max_sequence_length=32, hidden_size=32,
                                   intermediate_size=48, num_attention_heads=4,
                                   num_hidden_layers=2, expansion_rate=3, connection_type=kind))
        logits = model(tokens)
        logits.sum().backward()
        assert logits.shape == (2, 12, 40)
        assert all(p.grad is not None for p in model.parameters())
    cfg = TemplateConfig(vocab_size=40, seq_len=32, d_model=32, hidden_dim=48, num_heads=4,
                         num_layers=2)
    assert set(VARIANTS) == {"baseline", "kattention", "partial_kv", "xglu", "deglu", "springnet",
                             "tokenformer", "tokenformer_full", "mla", "relu2", "mixture_of_depth",
                             "hypersphere", "bitnet"}
    for variant in VARIANTS:
        model = build(variant, cfg)
        logits = model(tokens)
        assert logits.shape == (2, 12, 40)
        assert (model.auxiliary_loss is not None) == (variant in ("springnet", "mixture_of_depth"))
        logits.sum().backward()
    from experiments.misc.small_modules import XLinear as _X
    assert sum(isinstance(m, _X) for m in build("hypersphere", cfg).modules()) == 2 * 7
    from experiments.bitnet.bitnet import BitLinear
    assert sum(isinstance(m, BitLinear) for m in build("bitnet", cfg).modules()) == 2 * 7
    for name in ("griffin", "life"):
        result = main(["--model", name, "--steps", "30", "--batch", "8", "--seq-len", "48",
                       "--dim", "32", "--layers", "2", "--log-every", "0", "--device", "cpu"])
        assert result["last_loss"] < 0.9 * result["first_loss"], result
