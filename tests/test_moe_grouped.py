"""Grouped (stacked-weight) mixture of experts: routing, shared experts, balancing, optimizer
grouping and checkpoint shape recovery. Behaviour follows the reference suite
(tests/test_moe_grouped.py:33-463); the auxiliary loss and capacity factor are extensions."""

from __future__ import annotations

import pytest
import torch

from helpers import tiny_llama
from ohara_b200.chat_engine import config_from_state_dict
from ohara_b200.models.llama import Config, Llama
from ohara_b200.modules.moe import apply_qb_update, expert_load, maximal_violation
from ohara_b200.modules.moe_grouped import GroupedMoE
from ohara_b200.modules.routing import load_balance_aux_loss
from ohara_b200.optimizer import build_adamh, build_muon_adamw, build_muonh_adamh


def layer(**overrides) -> GroupedMoE:
    torch.manual_seed(0)
    settings = dict(dim=16, hidden_dim=24, num_experts=8, num_experts_per_tok=2, num_shared_experts=1)
    settings.update(overrides)
    module = GroupedMoE(**settings)
    with torch.no_grad():  # the down projections start at zero; give them something to do
        module.w_down.normal_(std=0.1)
        if module.num_shared_experts:
            module.shared_down.weight.normal_(std=0.1)
    return module


def test_stacked_parameters_and_zero_initialised_output():
    fresh = GroupedMoE(16, 24, num_experts=8, num_experts_per_tok=2, num_shared_experts=2)
    assert fresh.w_gate.shape == fresh.w_up.shape == (8, 16, 24) and fresh.w_down.shape == (8, 24, 16)
    assert fresh.shared_up.weight.shape == (48, 16), "shared experts widen one MLP"
    assert not hasattr(GroupedMoE(16, 24, 8, 2, num_shared_experts=0), "shared_gate")
    x = torch.randn(2, 5, 16, requires_grad=True)
    out = fresh(x)
    assert out.shape == x.shape and torch.all(out == 0)
    out.sum().backward()
    assert fresh.w_down.grad.abs().sum() > 0 and fresh.w_gate.grad.abs().sum() == 0
    assert fresh.router.weight.grad is None or fresh.router.weight.grad.abs().sum() == 0


def test_dispatch_matches_a_per_token_loop():
    moe = layer(num_shared_experts=0, gate_fn="softmax")
    x = torch.randn(3, 7, 16)
    flat = x.reshape(-1, 16)
    indices, weights, _, _ = moe._route(flat)
    expected = torch.zeros_like(flat)
    for t in range(flat.size(0)):
        for weight, e in zip(weights[t], indices[t]):
            h = torch.nn.functional.silu(flat[t] @ moe.w_gate[e]) * (flat[t] @ moe.w_up[e])
            expected[t] += weight * (h @ moe.w_down[e])
    assert torch.allclose(moe(x).reshape(-1, 16), expected, atol=1e-5)
    shared = layer(num_shared_experts=1, gate_fn="softmax")
    shared.load_state_dict(moe.state_dict(), strict=False)
    extra = shared(x) - moe(x)
    assert torch.allclose(extra.reshape(-1, 16), shared._shared(flat), atol=1e-5)


@pytest.mark.parametrize("gate, normalize, total", [("softmax", True, 1.0), ("sigmoid", True, 1.0),
                                                    ("sigmoid", False, None)])
def test_routing_weights(gate, normalize, total):
    moe = layer(gate_fn=gate, normalize_weights=normalize)
    indices, weights, logits, alpha = moe._route(torch.randn(32, 16))
    assert indices.shape == weights.shape == (32, 2) and weights.dtype == torch.float32
    assert all(len(set(row.tolist())) == 2 for row in indices), "k distinct experts per token"
    if total is None:
        assert torch.all((weights > 0) & (weights < 1)) and not torch.allclose(weights.sum(-1), torch.ones(32))
    else:
        assert torch.allclose(weights.sum(-1), torch.full((32,), total), atol=1e-6)
    assert alpha.shape == (32, 1), "the (k+1)-th biased score is the threshold"


def test_bias_steers_selection_without_touching_weights_or_gradients():
    moe = layer(gate_fn="sigmoid", normalize_weights=False)
    x = torch.randn(64, 16)
    before, _, logits, _ = moe._route(x)
    with torch.no_grad():
        moe.router_bias[3] = 100.0
    after, weights, _, _ = moe._route(x)
    assert torch.all((after == 3).any(-1)) and not torch.equal(before, after)
    assert torch.allclose(weights, torch.sigmoid(logits.gather(-1, after)))
    moe.train()
    moe(x.view(4, 16, 16)).sum().backward()
    assert not moe.router_bias.requires_grad and moe.router.weight.grad.abs().sum() > 0
    assert moe.w_gate.grad.abs().sum() > 0 and moe.shared_gate.weight.grad.abs().sum() > 0


def test_balancing_moves_a_mean_zero_bias_and_levels_the_load():
    moe = layer(num_experts=8).train()
    with torch.no_grad():
        moe.router.weight[0] = moe.router.weight[0].abs() + 1.0
    x = torch.randn(4, 64, 16).abs()
    moe(x)
    skewed = maximal_violation(moe.expert_load())
    for _ in range(30):
        moe(x)
        apply_qb_update(moe)
    assert moe.router_bias.abs().sum() > 0 and abs(float(moe.router_bias.mean())) < 1e-6
    moe.expert_load()
    moe(x)
    assert maximal_violation(expert_load(moe)[0]) < 0.5 * skewed

    off = layer(quantile_balancing=False).train()
    off(x)
    apply_qb_update(off)
    assert torch.all(off.router_bias == 0)
    assert int(off.expert_load().sum()) == 4 * 64 * 2, "load is recorded even without balancing"
    off.eval()
    off(x)
    assert int(off.expert_counts.sum()) == 0


def test_auxiliary_loss_and_capacity_extensions():
    logits = torch.zeros(8, 4)
    even = torch.arange(8).view(8, 1) % 4
    assert load_balance_aux_loss(logits, even, 4).item() == pytest.approx(1.0)
    lopsided = torch.zeros(8, 1, dtype=torch.long)
    peaked = torch.tensor([[4.0, 0, 0, 0]]).repeat(8, 1)
    assert load_balance_aux_loss(peaked, lopsided, 4) > 3.0
    moe = layer(aux_loss_coef=0.01, capacity_factor=0.5, num_shared_experts=0).train()
    moe(torch.randn(2, 32, 16))
    assert moe.aux_loss is not None and moe.aux_loss.requires_grad and moe.aux_loss > 0
    assert int(moe.dropped_pairs) > 0
    model = tiny_llama(64, moe_num_experts=4, moe_grouped=True, moe_aux_loss_coef=0.01).train()
    model(torch.randint(0, 64, (2, 8)))
    assert model.auxiliary_loss() > 0


def test_invalid_layers_are_refused():
    for bad in (dict(num_experts_per_tok=9), dict(num_experts_per_tok=8), dict(gate_fn="tanh"),
                dict(num_shared_experts=-1), dict(capacity_factor=0.0)):
        with pytest.raises(ValueError):
            layer(**bad)
    layer(num_experts_per_tok=8, quantile_balancing=False)
    base = dict(vocab_size=64, hidden_size=32, intermediate_size=64, max_sequence_length=16,
                num_hidden_layers=2, num_attention_heads=2)
    for bad in (dict(moe_num_shared_experts=1, moe_num_experts=4), dict(moe_grouped=True),
                dict(moe_normalize_weights=False, moe_num_experts=4)):
        with pytest.raises(ValueError):
            Llama(Config(**base, **bad))


def test_llama_keeps_the_coordinated_initialisation():
    model = tiny_llama(64, moe_num_experts=4, moe_grouped=True, moe_num_shared_experts=1,
                       init_style="nanochat")
    for block in model.layers:
        assert isinstance(block.ff, GroupedMoE)
        assert torch.all(block.ff.w_down == 0) and torch.all(block.ff.shared_down.weight == 0)
        assert block.ff.w_gate.abs().max() > 0 and torch.all(block.ff.router_bias == 0)


# -- optimizers --------------------------------------------------------------------------------------
def _moe_model():
    return tiny_llama(64, weight_tying=False, moe_num_experts=4, moe_grouped=True,
                      moe_num_shared_experts=1)


def test_expert_stacks_get_their_own_muon_groups():
    model = _moe_model()
    optimizer = build_muon_adamw(model, matrix_learning_rate=0.02)
    assigned = [p for group in optimizer.param_groups for p in group["params"]]
    assert len(assigned) == len(set(map(id, assigned))) == len(list(model.parameters()))
    expert_groups = [g for g in optimizer.param_groups
                     if any(p.dim() == 3 for p in g["params"])]
    assert expert_groups and all(g["kind"] == "muon" and g["lr"] == 0.02 for g in expert_groups)

    before = model.layers[0].ff.w_up.detach().clone()
    tokens = torch.randint(0, 64, (2, 9))
    loss = model(tokens[:, :-1], targets=tokens[:, 1:])
    loss.backward()
    optimizer.step()
    assert not torch.equal(model.layers[0].ff.w_up, before)
    assert all(torch.isfinite(p).all() for p in model.parameters())


@pytest.mark.parametrize("builder", [build_adamh, build_muonh_adamh])
def test_hyperspherical_steps_keep_every_expert_matrix_norm(builder):
    model = _moe_model()
    with torch.no_grad():
        for block in model.layers:
            block.ff.w_down.normal_(std=0.05)
    optimizer = builder(model)
    stack = model.layers[0].ff.w_gate
    norms = stack.detach().flatten(1).norm(dim=1).clone()
    for _ in range(2):
        tokens = torch.randint(0, 64, (2, 9))
        model(tokens[:, :-1], targets=tokens[:, 1:]).backward()
        optimizer.step()
        optimizer.zero_grad()
    assert not torch.allclose(stack.detach().flatten(1)[0], torch.zeros(1))
    assert torch.allclose(stack.detach().flatten(1).norm(dim=1), norms, rtol=1e-4)


# -- checkpoint shape recovery ----------------------------------------------------------------------
def test_configs_round_trip_through_state_dicts():
    grouped = tiny_llama(64, moe_num_experts=4, moe_grouped=True, moe_num_shared_experts=2,
                         moe_gate_fn="sigmoid", moe_normalize_weights=False, moe_experts_per_tok=3,
                         moe_layer_interval=2, num_hidden_layers=4)
    rebuilt = config_from_state_dict(grouped.state_dict(), moe_experts_per_tok=3,
                                     moe_gate_fn="sigmoid", moe_normalize_weights=False)
    for name in ("moe_num_experts", "moe_grouped", "moe_num_shared_experts", "moe_gate_fn",
                 "moe_normalize_weights", "moe_experts_per_tok", "moe_layer_interval",
                 "intermediate_size", "num_hidden_layers"):
        assert getattr(rebuilt, name) == getattr(grouped.config, name), name
    Llama(rebuilt).load_state_dict(grouped.state_dict())
    assert config_from_state_dict(grouped.state_dict()).moe_experts_per_tok == 2, "default top-k"

    looped = tiny_llama(64, moe_num_experts=3, moe_experts_per_tok=1)
    recovered = config_from_state_dict(looped.state_dict(), moe_experts_per_tok=1)
    assert recovered.moe_num_experts == 3 and not recovered.moe_grouped
    assert config_from_state_dict(tiny_llama(64).state_dict()).moe_num_experts == 0

    single = tiny_llama(64, moe_num_experts=4, moe_grouped=True, moe_layer_interval=3,
                        num_hidden_layers=3)
    mixed = config_from_state_dict(single.state_dict())
    assert mixed.moe_layer_interval == 3
    Llama(mixed).load_state_dict(single.state_dict())


# -- further behaviours of the reference suite (tests/test_moe_grouped.py:150-463) ---------------------
def test_gradients_reach_router_experts_and_shared_mlp_once_the_output_projection_is_nonzero():
    moe = layer()
    x = torch.randn(2, 6, 16, requires_grad=True)
    moe(x).square().sum().backward()
    for name in ("w_gate", "w_up", "w_down"):
        assert getattr(moe, name).grad.abs().sum() > 0, name
    assert moe.router.weight.grad.abs().sum() > 0
    assert moe.shared_gate.weight.grad.abs().sum() > 0 and x.grad.abs().sum() > 0
    assert not moe.router_bias.requires_grad and moe.router_bias.grad is None


def test_statistics_accumulate_only_in_training_and_disabled_balancing_keeps_a_zero_bias():
    moe = layer()
    x = torch.randn(4, 8, 16)
    moe.eval()
    moe(x)
    assert int(moe.expert_counts.sum()) == 0 and int(moe.qb_beta_count) == 0
    moe.train()
    moe(x)
    assert int(moe.expert_counts.sum()) == 4 * 8 * 2 and int(moe.qb_beta_count) == 1
    plain = layer(quantile_balancing=False)
    plain.train()
    for _ in range(3):
        plain(torch.randn(4, 8, 16))
        plain.apply_qb_update()
    assert torch.all(plain.router_bias == 0)


def test_model_level_helpers_see_grouped_layers_and_each_token_picks_distinct_experts():
    model = tiny_llama(40, moe_num_experts=4, moe_experts_per_tok=2, moe_grouped=True)
    model.train()
    model(torch.randint(0, model.config.vocab_size, (2, 8)))
    loads = expert_load(model, reset=False)
    assert len(loads) == model.config.num_hidden_layers
    assert all(int(c.sum()) == 2 * 8 * 2 for c in loads)
    assert maximal_violation(loads[0]) >= 0.0
    apply_qb_update(model)                                    # walks the grouped layers too
    assert any(bool((b.ff.router_bias != 0).any()) for b in model.layers)
    moe = layer(num_experts_per_tok=3)
    indices, _, _, _ = moe._route(torch.randn(50, 16))
    assert all(len(set(row.tolist())) == 3 for row in indices)


def test_llama_refuses_grouped_only_options_without_the_grouped_layer():
    with pytest.raises(ValueError):
        Llama(Config(moe_num_experts=4, moe_grouped=False, moe_num_shared_experts=1))
    with pytest.raises(ValueError):
        Llama(Config(moe_num_experts=0, moe_grouped=True))


def test_checkpoint_shapes_recover_mixed_dense_and_moe_layouts_and_default_routing_choices():
    mixed = tiny_llama(40, moe_num_experts=4, moe_experts_per_tok=2, moe_grouped=True,
                       moe_layer_interval=2, moe_num_shared_experts=2, num_hidden_layers=4)
    cfg = config_from_state_dict(mixed.state_dict())
    assert (cfg.moe_num_experts, cfg.moe_layer_interval, cfg.moe_num_shared_experts) == (4, 2, 2)
    assert cfg.moe_grouped and cfg.moe_experts_per_tok == 2            # the default when not given
    rebuilt = Llama(cfg)
    rebuilt.load_state_dict(mixed.state_dict())
    single = tiny_llama(40, moe_num_experts=4, moe_grouped=True, moe_layer_interval=3,
                        num_hidden_layers=3)                           # one MoE layer out of three
    assert config_from_state_dict(single.state_dict()).moe_layer_interval == 3
    chosen = config_from_state_dict(mixed.state_dict(), moe_experts_per_tok=3, moe_gate_fn="sigmoid",
                                    moe_normalize_weights=False)
    assert (chosen.moe_experts_per_tok, chosen.moe_gate_fn, chosen.moe_normalize_weights) == (
        3, "sigmoid", False)
    dense = config_from_state_dict(tiny_llama(40).state_dict())
    assert dense.moe_num_experts == 0
    looped = config_from_state_dict(tiny_llama(40, moe_num_experts=4, moe_experts_per_tok=2).state_dict())
    assert looped.moe_num_experts == 4 and not looped.moe_grouped


def test_a_muon_step_moves_the_expert_stacks_and_keeps_them_finite():
    model = tiny_llama(40, moe_num_experts=4, moe_experts_per_tok=2, moe_grouped=True)
    optimizer = build_muon_adamw(model)
    listed = [p for g in optimizer.param_groups for p in g["params"]]
    assert {id(p) for p in listed} == {id(p) for p in model.parameters()}
    before = model.layers[0].ff.w_down.detach().clone()
    tokens = torch.randint(0, model.config.vocab_size, (2, 9))
    for _ in range(2):
        logits = model(tokens[:, :-1])
        torch.nn.functional.cross_entropy(logits.flatten(0, 1), tokens[:, 1:].flatten()).backward()
        optimizer.step()
        optimizer.zero_grad()
    after = model.layers[0].ff.w_down.detach()
    assert torch.isfinite(after).all() and not torch.equal(after, before)
