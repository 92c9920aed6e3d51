"""Llama model: validation, state-dict layout, cached decoding, accounting, initialisation."""

import pytest
import torch

from ohara_b200.models.llama import Config, Llama


def tiny(**kw):
    base = dict(vocab_size=97, max_sequence_length=32, hidden_size=64, intermediate_size=96,
                num_attention_heads=4, num_hidden_layers=2, dropout=0.0)
    base.update(kw)
    return Config(**base)


@pytest.mark.parametrize(
    "field,value",
    [("vocab_size", 1), ("hidden_size", 0), ("intermediate_size", 0), ("num_attention_heads", 3),
     ("max_sequence_length", 1), ("num_key_value_heads", 3), ("dropout", 1.0),
     ("init_style", "weird"), ("moe_layer_interval", 0), ("moe_gate_fn", "tanh")],
)
def test_config_rejections(field, value):
    with pytest.raises(ValueError):
        Llama(tiny(**{field: value}))


def test_more_config_rejections():
    with pytest.raises(ValueError):
        Llama(tiny(init_style="nanochat", weight_tying=True))
    with pytest.raises(ValueError):
        Llama(tiny(moe_grouped=True))
    with pytest.raises(ValueError):
        Llama(tiny(moe_num_experts=4, moe_num_shared_experts=1))
    with pytest.raises(ValueError):
        Llama(tiny(moe_num_experts=4, moe_normalize_weights=False))


def test_state_dict_layout_matches_reference_names():
    model = Llama(tiny(num_key_value_heads=2))
    keys = set(model.state_dict())
    for name in ["token_emb.weight", "vocab_proj.weight", "norm.weight", "freq_cos", "freq_sin",
                 "layers.0.attn.key.weight", "layers.0.attn.query.weight",
                 "layers.0.attn.value.weight", "layers.0.attn.proj.weight",
                 "layers.1.ff.up.weight", "layers.1.ff.down.weight", "layers.1.ff.gate.weight",
                 "layers.0.norm1.weight", "layers.0.norm2.weight"]:
        assert name in keys
    sd = model.state_dict()
    assert sd["layers.0.attn.key.weight"].shape == (2 * 16, 64)
    assert sd["freq_cos"].shape == (64, 8)  # 2 x context, head_dim / 2


def test_weight_tying_shares_storage():
    model = Llama(tiny(weight_tying=True))
    assert model.token_emb.weight is model.vocab_proj.weight
    assert model.num_scaling_params()["lm_head"] == 0


@pytest.mark.parametrize("kv_heads", [0, 2, 1])
def test_cached_decode_matches_full_forward(kv_heads):
    torch.manual_seed(0)
    model = Llama(tiny(num_key_value_heads=kv_heads)).eval()
    ids = torch.randint(0, 97, (2, 20))
    full = model(ids)
    cache = model.build_kv_cache(2)
    parts = [model(ids[:, :7], cache, 0), model(ids[:, 7:15], cache, 7)]
    for pos in range(15, 20):
        parts.append(model(ids[:, pos : pos + 1], cache, torch.tensor(pos)))
    assert torch.allclose(torch.cat(parts, dim=1), full, atol=1e-5)


def test_cache_and_position_errors():
    model = Llama(tiny()).eval()
    ids = torch.randint(0, 97, (1, 8))
    cache = model.build_kv_cache(1)
    with pytest.raises(ValueError):
        model(ids, cache)  # missing position
    with pytest.raises(ValueError):
        model(ids, None, 3)  # position without cache
    with pytest.raises(ValueError):
        model(ids, cache[:1], 0)
    with pytest.raises(ValueError):
        model(torch.randint(0, 97, (1, 40)))
    with pytest.raises(ValueError):
        model(ids[0])
    model(ids, cache, 0)
    with pytest.raises(ValueError):
        model(ids, cache, 3)  # non-sequential write
    with pytest.raises(ValueError):
        model.build_kv_cache(0)


def test_loss_sum_equals_logits_cross_entropy():
    torch.manual_seed(1)
    model = Llama(tiny())
    ids = torch.randint(0, 97, (3, 17))
    x, y = ids[:, :-1], ids[:, 1:].clone()
    y[0, :5] = -1
    logits = model(x)
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, 97), y.reshape(-1), ignore_index=-1,
                                            reduction="sum")
    assert torch.allclose(model.loss_sum(x, y), ref, rtol=1e-5)
    assert torch.allclose(model(x, targets=y, loss_scale=0.5), 0.5 * ref, rtol=1e-5)


def test_flops_and_param_accounting():
    model = Llama(tiny())
    groups = model.num_scaling_params()
    assert groups["total"] == sum(p.numel() for p in model.parameters())
    assert groups["effective"] == groups["transformer_matrices"] + groups["lm_head"]
    per_block = 4 * 64 * 64 + 3 * 64 * 96
    assert model.active_matmul_parameters() == 2 * per_block
    expected = 6 * (2 * per_block + 97 * 64) + 12 * 2 * 4 * 16 * 32
    assert model.estimate_flops() == float(expected)
    with pytest.raises(ValueError):
        model.estimate_flops(100)


def test_moe_active_parameters_count_k_of_e():
    cfg = tiny(moe_num_experts=8, moe_experts_per_tok=2, moe_grouped=True, moe_num_shared_experts=1)
    model = Llama(cfg)
    attn = 4 * 64 * 64
    per_expert = 64 * 96 * 3
    assert model.active_matmul_parameters() == 2 * (attn + per_expert * 3 + 8 * 64)
    loop = Llama(tiny(moe_num_experts=4, moe_experts_per_tok=2))
    assert loop.active_matmul_parameters() == 2 * (attn + per_expert * 2 + 4 * 64)


def test_nanochat_init_zeroes_output_projections():
    model = Llama(tiny(init_style="nanochat"))
    for block in model.layers:
        assert float(block.attn.proj.weight.abs().sum()) == 0.0
        assert float(block.ff.down.weight.abs().sum()) == 0.0
    assert 0.6 < float(model.token_emb.weight.std()) < 1.0
    assert float(model.vocab_proj.weight.std()) < 0.01
    # With zero output projections every block is the identity on the residual stream.
    ids = torch.randint(0, 97, (1, 8))
    hidden = model.forward_hidden(ids)
    emb = model.norm(model.token_emb(ids))
    assert torch.allclose(hidden, emb, atol=1e-6)


def test_rope_theta_changes_tables():
    a = Llama(tiny(rope_theta=10000.0))
    b = Llama(tiny(rope_theta=500000.0))
    assert not torch.allclose(a.freq_cos, b.freq_cos)


def test_from_pretrained_not_implemented():
    with pytest.raises(NotImplementedError):
        Llama.from_pretrained("x")
