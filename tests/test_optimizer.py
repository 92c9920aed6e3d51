"""Optimizers: partitioning, AdamW equivalence, Muon maths and resume, hyperspherical variants."""

import io
import math

import pytest
import torch

from ohara_b200.models.llama import Config, Llama
from ohara_b200.optimizer import (
    POLAR_EXPRESS_COEFFICIENTS,
    MuonAdamW,
    _hypersphere_update_,
    _hypersphere_update_stacked_,
    _partition_llama_parameters,
    _polar_express,
    build_adamh,
    build_adamw,
    build_muon_adamw,
    build_muonh_adamh,
)


def small(**kw):
    base = dict(vocab_size=61, max_sequence_length=16, hidden_size=32, intermediate_size=48,
                num_attention_heads=2, num_hidden_layers=2, dropout=0.0)
    base.update(kw)
    return Llama(Config(**base))


def loss_and_backward(model, seed=0):
    gen = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 61, (4, 13), generator=gen)
    loss = model.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
    loss.backward()
    return float(loss)


def test_build_adamw_groups_and_validation():
    model = small()
    opt = build_adamw(model, learning_rate=1e-3, weight_decay=0.1)
    decay, no_decay = opt.param_groups
    assert all(p.ndim >= 2 for p in decay["params"]) and decay["weight_decay"] == 0.1
    assert all(p.ndim < 2 for p in no_decay["params"]) and no_decay["weight_decay"] == 0.0
    with pytest.raises(ValueError):
        build_adamw(model, learning_rate=0.0, weight_decay=0.1)
    with pytest.raises(ValueError):
        build_adamw(model, learning_rate=1e-3, weight_decay=-1.0)


def test_partition_is_complete_and_handles_tying_and_experts():
    model = small(moe_num_experts=4, moe_grouped=True, moe_num_shared_experts=1)
    part = _partition_llama_parameters(model, "test")
    assigned = part.embedding + part.unembedding + part.matrix + part.stacked_matrix + part.scalar
    assert {id(p) for p in assigned} == {id(p) for p in model.parameters()}
    assert len(part.stacked_matrix) == 2 * 3 and all(p.ndim == 3 for p in part.stacked_matrix)
    tied = small(weight_tying=True)
    assert _partition_llama_parameters(tied, "test").unembedding == []
    with pytest.raises(TypeError):
        _partition_llama_parameters(torch.nn.Linear(2, 2), "test")


def test_muon_group_metadata():
    model = small()
    opt = build_muon_adamw(model, matrix_learning_rate=0.02)
    names = [g["name"] for g in opt.param_groups]
    assert names[:3] == ["unembedding", "embedding", "norms_and_scalars"]
    for group in opt.param_groups:
        assert group["initial_lr"] == group["lr"]
        assert math.isclose(group["lr_scale"], group["lr"] / 0.02)
        assert group["kind"] in ("adamw", "muon")
    width = math.sqrt(768 / 32)
    assert math.isclose(opt.param_groups[0]["lr"], 0.008 * width)
    muon = [g for g in opt.param_groups if g["kind"] == "muon"]
    assert all(len({p.shape for p in g["params"]}) == 1 for g in muon)
    assert all(g["name"].startswith("matrix_") for g in muon)


def test_hybrid_adamw_matches_torch_adamw():
    torch.manual_seed(0)
    w1 = torch.randn(8, 5, requires_grad=True)
    w2 = w1.detach().clone().requires_grad_()
    ours = MuonAdamW([{"kind": "adamw", "params": [w1], "lr": 1e-2, "betas": (0.9, 0.95),
                       "eps": 1e-8, "weight_decay": 0.1}])
    ref = torch.optim.AdamW([w2], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(6):
        g = torch.randn(8, 5)
        w1.grad, w2.grad = g.clone(), g.clone()
        ours.step()
        ref.step()
    assert torch.allclose(w1, w2, atol=1e-6)


def test_polar_express_orthogonalises_both_orientations():
    torch.manual_seed(0)
    for shape in [(3, 24, 16), (2, 16, 40)]:
        x = _polar_express(torch.randn(*shape), 5)
        gram = x.mT @ x if shape[1] > shape[2] else x @ x.mT
        eye = torch.eye(gram.shape[-1])
        assert (gram - eye).abs().max() < 0.3
    with pytest.raises(ValueError):
        _polar_express(torch.randn(4, 4), 5)
    with pytest.raises(ValueError):
        _polar_express(torch.randn(1, 4, 4), 6)
    assert len(POLAR_EXPRESS_COEFFICIENTS) == 5


def test_muon_step_matches_written_out_update():
    torch.manual_seed(0)
    params = [torch.randn(12, 8, requires_grad=True) for _ in range(3)]
    before = torch.stack([p.detach().clone() for p in params])
    grads = torch.stack([torch.randn(12, 8) for _ in range(3)])
    for p, g in zip(params, grads):
        p.grad = g.clone()
    opt = MuonAdamW([{"kind": "muon", "params": params, "lr": 0.05, "weight_decay": 0.1,
                      "momentum": 0.9, "beta2": 0.8, "ns_steps": 5}])
    opt.step()
    buf = (1 - 0.9) * grads
    u = grads + 0.9 * (buf - grads)
    x = _polar_express(u, 5)
    v = x.square().mean(dim=-1, keepdim=True)  # rows >= cols -> reduce the last dim
    n0 = (v.sum(dim=(-2, -1), keepdim=True) * 8).sqrt()
    s = (1 - 0.8) * v
    rho = s.clamp_min(1e-10).rsqrt()
    n1 = ((v * 8) * rho.square()).sum(dim=(-2, -1), keepdim=True).sqrt()
    x = x * rho * (n0 / n1.clamp_min(1e-10))
    lr = 0.05 * math.sqrt(12 / 8)
    expected = before - lr * x - lr * 0.1 * before * ((x * before) >= 0)
    assert torch.allclose(torch.stack([p.detach() for p in params]), expected, atol=1e-5)
    state = opt.state[params[0]]
    assert state["momentum_buffer"].shape == (3, 12, 8)
    assert state["second_momentum_buffer"].shape == (3, 12, 1)


def test_muon_requires_all_grads_and_same_shapes():
    a, b = torch.randn(4, 4, requires_grad=True), torch.randn(4, 4, requires_grad=True)
    opt = MuonAdamW([{"kind": "muon", "params": [a, b], "lr": 0.1}])
    a.grad = torch.randn(4, 4)
    opt.param_groups[0].update(momentum=0.95, ns_steps=5, beta2=0.9, weight_decay=0.0)
    with pytest.raises(RuntimeError):
        opt.step()
    with pytest.raises(ValueError):
        MuonAdamW([{"kind": "muon", "params": [a, torch.randn(4, 5, requires_grad=True)], "lr": 0.1}])
    with pytest.raises(ValueError):
        MuonAdamW([{"kind": "sgd", "params": [a], "lr": 0.1}])
    with pytest.raises(ValueError):
        MuonAdamW([{"kind": "adamw", "params": [a], "lr": 0.1, "hypersphere": True,
                    "weight_decay": 0.1}])
    with pytest.raises(ValueError):
        MuonAdamW([])


def _serialized(state):
    buffer = io.BytesIO()
    torch.save(state, buffer)
    buffer.seek(0)
    return torch.load(buffer, weights_only=False)


@pytest.mark.parametrize("builder", [build_muon_adamw, build_muonh_adamh, build_adamh])
def test_checkpoint_resume_reproduces_trajectory(builder):
    torch.manual_seed(0)
    model_a = small()
    opt_a = builder(model_a)
    for step in range(2):
        loss_and_backward(model_a, step)
        opt_a.step()
        opt_a.zero_grad()
    model_b = small()
    model_b.load_state_dict(_serialized(model_a.state_dict()))
    opt_b = builder(model_b)
    opt_b.load_state_dict(_serialized(opt_a.state_dict()))
    for step in range(2, 4):
        for model, opt in ((model_a, opt_a), (model_b, opt_b)):
            loss_and_backward(model, step)
            opt.step()
            opt.zero_grad()
    for pa, pb in zip(model_a.parameters(), model_b.parameters()):
        assert torch.equal(pa, pb)


def test_hypersphere_updates_preserve_norm_and_match_each_other():
    torch.manual_seed(0)
    params = [torch.randn(6, 4) for _ in range(3)]
    dirs = [torch.randn(6, 4) for _ in range(3)]
    norms = [p.norm().item() for p in params]
    stacked = torch.stack([p.clone() for p in params])
    _hypersphere_update_(params, dirs, 0.1)
    _hypersphere_update_stacked_(stacked, torch.stack(dirs), 0.1)
    for p, n, s in zip(params, norms, stacked):
        assert math.isclose(p.norm().item(), n, rel_tol=1e-5)
        assert torch.allclose(p, s, atol=1e-6)
    # scale invariance: only the direction of the update matters
    q1, q2 = torch.randn(5, 5), None
    q2 = q1.clone()
    d = torch.randn(5, 5)
    _hypersphere_update_([q1], [d], 0.05)
    _hypersphere_update_([q2], [d * 37.0], 0.05)
    assert torch.allclose(q1, q2, atol=1e-6)


def test_hyperspherical_builders_assign_groups_and_hold_norms():
    model = small()
    opt = build_muonh_adamh(model)
    kinds = {g["name"].split("_")[0] for g in opt.param_groups}
    assert {"muonh", "adamh", "embedding"} <= kinds
    assert all(g["weight_decay"] == 0.0 for g in opt.param_groups)
    matrices = [p for g in opt.param_groups if g.get("hypersphere") for p in g["params"]]
    norms = [p.norm().item() for p in matrices]
    first = loss_and_backward(model, 0)
    opt.step()
    opt.zero_grad()
    for step in range(1, 8):
        last = loss_and_backward(model, 0)
        opt.step()
        opt.zero_grad()
    assert last < first
    for p, n in zip(matrices, norms):
        assert math.isclose(p.norm().item(), n, rel_tol=1e-4)
    adamh = build_adamh(small())
    assert any(g["name"].startswith("adamh_") and g.get("hypersphere") for g in adamh.param_groups)


def test_training_lowers_loss_with_muon():
    torch.manual_seed(0)
    model = small()
    opt = build_muon_adamw(model)
    first = loss_and_backward(model, 0)
    opt.step()
    opt.zero_grad()
    for _ in range(10):
        last = loss_and_backward(model, 0)
        opt.step()
        opt.zero_grad()
    assert last < 0.7 * first


def test_stacked_expert_tensors_go_to_muon():
    model = small(moe_num_experts=4, moe_grouped=True)
    opt = build_muon_adamw(model)
    experts = [g for g in opt.param_groups if g["name"].startswith("expert_")]
    assert len(experts) == 6 and all(g["kind"] == "muon" and g["params"][0].ndim == 3 for g in experts)
    with torch.no_grad():
        for block in model.layers:
            block.ff.w_down.normal_(std=0.02)
    loss_and_backward(model, 0)
    before = model.layers[0].ff.w_gate.detach().clone()
    opt.step()
    assert not torch.equal(before, model.layers[0].ff.w_gate)
