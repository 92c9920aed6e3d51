"""AdamH and MuonH, the constant-norm optimizers: properties of the projection rule, validation of
hyperspherical groups, what the two builders put where, and training behaviour (the contract the
reference pins in tests/test_optimizers_hypersphere.py)."""

import io

import pytest
import torch
import torch.nn.functional as F

from ohara_b200.models.llama import Config, Llama
from ohara_b200.optimizer import (MuonAdamW, _hypersphere_update_, _hypersphere_update_stacked_,
                                  build_adamh, build_muonh_adamh)

BUILDERS = [build_adamh, build_muonh_adamh]


def _model(**extra) -> Llama:
    torch.manual_seed(7)
    return Llama(Config(vocab_size=48, max_sequence_length=24, hidden_size=48, intermediate_size=96,
                        num_attention_heads=4, num_hidden_layers=2, dropout=0.0,
                        weight_tying=False, **extra))


def _fit(model, optimizer, steps):
    generator = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, 48, (4, 13), generator=generator)
    trace = []
    for _ in range(steps):
        loss = F.cross_entropy(model(tokens[:, :-1]).flatten(0, 1), tokens[:, 1:].flatten())
        optimizer.zero_grad(set_to_none=True)
        loss.backward()
        optimizer.step()
        trace.append(float(loss.detach()))
    return trace


def _group_of(optimizer, parameter):
    return next(g for g in optimizer.param_groups if any(p is parameter for p in g["params"]))


# -- the update rule ---------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(5, 3), (7, 7), (2, 9)])
def test_update_keeps_the_frobenius_norm(shape):
    torch.manual_seed(0)
    weights = [torch.randn(shape) * s for s in (0.3, 4.0)]
    norms = [w.norm().item() for w in weights]
    _hypersphere_update_(weights, [torch.randn(shape) for _ in weights], 0.25)
    assert [w.norm().item() for w in weights] == pytest.approx(norms, rel=1e-6)


def test_only_the_direction_of_the_update_matters():
    torch.manual_seed(0)
    start = [torch.randn(4, 6), torch.randn(4, 6)]
    step = [torch.randn(4, 6), torch.randn(4, 6)]
    small, large = [w.clone() for w in start], [w.clone() for w in start]
    _hypersphere_update_(small, [u * 1e-3 for u in step], 0.05)
    _hypersphere_update_(large, [u * 5e2 for u in step], 0.05)
    for a, b in zip(small, large):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rate", [0.005, 0.03, 0.15])
def test_learning_rate_is_the_relative_length_of_the_step(rate):
    torch.manual_seed(0)
    weight = torch.randn(12, 20)
    moved = [weight.clone()]
    _hypersphere_update_(moved, [torch.randn(12, 20)], rate)
    relative = float((moved[0] - weight).norm() / weight.norm())
    assert 0.7 * rate <= relative <= rate * (1 + 1e-3)      # the chord is never longer than lr


def test_stacked_form_equals_the_per_tensor_form_and_zero_updates_do_nothing():
    torch.manual_seed(0)
    weights = [torch.randn(5, 8) for _ in range(4)]
    updates = [torch.randn(5, 8) for _ in range(4)]
    stacked = torch.stack(weights).clone()
    _hypersphere_update_stacked_(stacked, torch.stack(updates), 0.08)
    listed = [w.clone() for w in weights]
    _hypersphere_update_(listed, updates, 0.08)
    torch.testing.assert_close(stacked, torch.stack(listed), rtol=1e-6, atol=1e-6)
    frozen = [w.clone() for w in weights]
    _hypersphere_update_(frozen, [torch.zeros(5, 8) for _ in weights], 0.08)
    torch.testing.assert_close(torch.stack(frozen), torch.stack(weights), rtol=1e-6, atol=1e-6)
    _hypersphere_update_([], [], 0.1)                          # an empty group is fine


# -- group validation --------------------------------------------------------------------------------
def _spherical_group(parameter, **changes):
    group = {"kind": "adamw", "hypersphere": True, "params": [parameter], "lr": 0.02,
             "betas": (0.9, 0.95), "eps": 1e-8, "weight_decay": 0.0}
    group.update(changes)
    return group


def test_spherical_groups_take_neither_weight_decay_nor_vectors():
    matrix = torch.nn.Parameter(torch.randn(3, 3))
    MuonAdamW([_spherical_group(matrix)])                      # the valid form constructs
    with pytest.raises(ValueError, match="weight_decay=0"):
        MuonAdamW([_spherical_group(matrix, weight_decay=0.01)])
    with pytest.raises(ValueError, match="matrix parameters only"):
        MuonAdamW([_spherical_group(torch.nn.Parameter(torch.randn(3)))])


# -- builders ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("builder", BUILDERS)
def test_builders_cover_every_parameter_once_without_decay_on_the_sphere(builder):
    model = _model()
    optimizer = builder(model)
    listed = [p for g in optimizer.param_groups for p in g["params"]]
    assert len(listed) == len({id(p) for p in listed})
    assert {id(p) for p in listed} == {id(p) for p in model.parameters()}
    for group in optimizer.param_groups:
        if group.get("hypersphere"):
            assert group["weight_decay"] == 0.0 and all(p.ndim >= 2 for p in group["params"])
    with pytest.raises(ValueError, match="positive"):
        builder(_model(), learning_rate=0.0)


def test_adamh_and_muonh_place_head_hidden_matrices_embedding_and_gains():
    model = _model()
    adamh = build_adamh(model)
    assert _group_of(adamh, model.vocab_proj.weight).get("hypersphere") is True
    assert all(g["weight_decay"] == 0.0 for g in adamh.param_groups)
    muonh = build_muonh_adamh(model, learning_rate=0.04)
    hidden = _group_of(muonh, model.layers[1].ff.down.weight)
    assert (hidden["kind"], hidden["hypersphere"]) == ("muon", True)
    head = _group_of(muonh, model.vocab_proj.weight)            # a matrix, but not orthogonalised
    assert (head["kind"], head["hypersphere"]) == ("adamw", True)
    for plain in (model.token_emb.weight, model.layers[0].norm2.weight, model.norm.weight):
        group = _group_of(muonh, plain)
        assert group["kind"] == "adamw" and not group.get("hypersphere", False)
    spherical = [g for g in muonh.param_groups if g.get("hypersphere")]
    assert len(spherical) >= 2 and {g["lr"] for g in spherical} == {0.04}   # one rate for both


# -- training ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("builder", BUILDERS)
def test_training_lowers_the_loss_and_matrices_stay_on_their_spheres(builder):
    model = _model()
    radius = {n: p.detach().norm().item() for n, p in model.named_parameters()
              if p.ndim == 2 and "token_emb" not in n}
    trace = _fit(model, builder(model), 25)
    assert trace[-1] < trace[0]
    now = dict(model.named_parameters())
    for name, value in radius.items():
        assert now[name].detach().norm().item() == pytest.approx(value, rel=1e-4), name


def test_learning_rate_sets_how_far_matrices_rotate():
    cosine = {}
    for rate in (1e-8, 0.2):
        model = _model()
        before = model.layers[0].attn.key.weight.detach().clone()
        _fit(model, build_muonh_adamh(model, learning_rate=rate), 15)
        after = model.layers[0].attn.key.weight.detach()
        cosine[rate] = float((after * before).sum() / (after.norm() * before.norm()))
    assert cosine[1e-8] > 0.999 and cosine[0.2] < 0.9


def _through_a_file(state):
    """A real resume loads from disk; loading in process would share momentum tensors."""
    buffer = io.BytesIO()
    torch.save(state, buffer)
    buffer.seek(0)
    return torch.load(buffer, weights_only=False)


@pytest.mark.parametrize("builder", BUILDERS)
def test_resumed_run_repeats_the_uninterrupted_one(builder):
    model = _model()
    optimizer = builder(model)
    _fit(model, optimizer, 3)
    twin = _model()
    twin.load_state_dict(_through_a_file(model.state_dict()))
    twin_optimizer = builder(twin)
    twin_optimizer.load_state_dict(_through_a_file(optimizer.state_dict()))
    assert _fit(model, optimizer, 3) == pytest.approx(_fit(twin, twin_optimizer, 3), rel=1e-6, abs=1e-7)
