"""Activation checkpointing of the Llama blocks: same loss and gradients as the plain step, less
saved activation memory, and routers that count every token once."""

import pytest
import torch

from ohara_b200 import Config, Llama
from ohara_b200.modules.routing import expert_load


def _model(moe: bool) -> Llama:
    torch.manual_seed(3)
    extra = dict(moe_num_experts=8, moe_experts_per_tok=2, moe_grouped=True,
                 moe_num_shared_experts=1, moe_aux_loss_coef=0.01) if moe else {}
    return Llama(Config(vocab_size=61, max_sequence_length=32, hidden_size=32, intermediate_size=48,
                        num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3,
                        dropout=0.0, **extra))


def _step(model: Llama, tokens: torch.Tensor):
    model.zero_grad(set_to_none=True)
    loss = model(tokens[:, :-1], targets=tokens[:, 1:])
    loss.backward()
    return loss.detach(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("moe", [False, True])
def test_checkpointed_step_matches_plain_step(moe):
    tokens = torch.randint(0, 61, (2, 17), generator=torch.Generator().manual_seed(0))
    plain, recomputed = _model(moe), _model(moe).enable_activation_checkpointing()
    plain.train(), recomputed.train()
    loss_a, grads_a = _step(plain, tokens)
    loss_b, grads_b = _step(recomputed, tokens)
    torch.testing.assert_close(loss_a, loss_b, rtol=1e-6, atol=1e-6)
    assert grads_a.keys() == grads_b.keys()
    for name in grads_a:
        torch.testing.assert_close(grads_a[name], grads_b[name], rtol=1e-5, atol=1e-6, msg=name)
    if moe:
        # the second forward pass of every block must not count its tokens again
        for a, b in zip(expert_load(plain), expert_load(recomputed)):
            assert torch.equal(a, b)
            assert int(a.sum()) == 2 * 16 * 2


def test_checkpointing_saves_fewer_tensors():
    tokens = torch.randint(0, 61, (2, 17), generator=torch.Generator().manual_seed(0))
    saved = {}
    for name, model in (("plain", _model(False)), ("recomputed", _model(False).enable_activation_checkpointing())):
        model.train()
        total = 0

        def pack(tensor):
            nonlocal total
            total += tensor.numel() * tensor.element_size()
            return tensor

        with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
            loss = model(tokens[:, :-1], targets=tokens[:, 1:])
        loss.backward()
        saved[name] = total
    assert saved["recomputed"] < 0.5 * saved["plain"], saved


def test_inference_and_eval_ignore_the_flag():
    model = _model(False).enable_activation_checkpointing()
    tokens = torch.randint(0, 61, (1, 9))
    model.eval()
    with torch.no_grad():
        a = model(tokens)
    model.activation_checkpointing = False
    with torch.no_grad():
        b = model(tokens)
    assert torch.equal(a, b)


def test_engine_flag_switches_it_on():
    from ohara_b200 import OharaEngine
    from ohara_b200.runtime import EngineConfig

    engine = OharaEngine(EngineConfig(activation_checkpointing=True))
    model = engine.prepare(_model(False))
    assert model.activation_checkpointing
    with pytest.raises(ValueError):
        OharaEngine(EngineConfig(activation_checkpointing=True)).prepare(torch.nn.Linear(4, 4))
