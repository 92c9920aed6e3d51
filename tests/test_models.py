"""Smoke and consistency tests of the model zoo and adapters."""

import pytest
import torch

from ohara_b200.models import gemma, gpt, mamba, phi, retnet, roformer, transformer
from ohara_b200.adaptor.dora import DoRALinear, mark_dora_as_trainable, merge_dora, replace_with_dora
from ohara_b200.adaptor.lora import LoRALinear, mark_lora_as_trainable, merge_lora, replace_with_lora


def ids(vocab=65, batch=2, seq=12):
    return torch.randint(0, vocab, (batch, seq))


@pytest.mark.parametrize("mlp", ["mlp", "swiglu", "geglu"])
def test_gpt_forward(mlp):
    model = gpt.GPT(gpt.Config(mlp=mlp, dropout=0.0))
    out = model(ids())
    assert out.shape == (2, 12, 65) and torch.isfinite(out).all()
    with pytest.raises(ValueError):
        gpt.GPT(gpt.Config(mlp="nope"))
    with pytest.raises(ValueError):
        model(torch.randint(0, 65, (1, 100)))


def test_roformer_retnet_gemma_transformer_forward():
    assert roformer.RoFormer(roformer.Config(dropout=0.0))(ids()).shape == (2, 12, 65)
    assert retnet.RetNet(retnet.Config(dropout=0.0))(ids()).shape == (2, 12, 65)
    g = gemma.GemmaConfig(vocab_size=65, max_sequence_length=32, hidden_size=64,
                          num_attention_heads=4, num_key_value_heads=1, num_hidden_layers=2)
    g.intermediate_size = 96
    model = gemma.Gemma(g)
    assert model(ids()).shape == (2, 12, 65)
    assert model.token_emb.weight is model.vocab_proj.weight
    cfg = transformer.Config(vocab_size=65, seq_len=32, d_model=64, hidden_dim=96, num_heads=4,
                             num_kv_heads=2, dropout=0.0)
    assert transformer.Transformer(cfg)(ids()).shape == (2, 12, 65)
    with pytest.raises(ValueError):
        roformer.RoFormer(roformer.Config(d_model=12, num_heads=4))


def test_causality_of_attention_models():
    torch.manual_seed(0)
    model = roformer.RoFormer(roformer.Config(dropout=0.0)).eval()
    a = ids()
    b = a.clone()
    b[:, -1] = (b[:, -1] + 1) % 65
    assert torch.allclose(model(a)[:, :-1], model(b)[:, :-1], atol=1e-5)


def test_modeling_lm_save_and_load(tmp_path):
    cfg = transformer.Config(vocab_size=65, seq_len=32, d_model=32, hidden_dim=48, num_heads=2,
                             num_layers=1, dropout=0.0)
    model = transformer.ModelingLM(cfg).eval()
    x = ids()
    model.save_pretrained(tmp_path / "lm")
    loaded = transformer.ModelingLM.from_pretrained(tmp_path / "lm").eval()
    assert torch.allclose(model(x), loaded(x), atol=1e-6)


def test_phi_cached_decode_matches_full():
    torch.manual_seed(0)
    cfg = phi.PhiConfig(vocab_size=65, max_sequence_length=32, hidden_size=64,
                        num_attention_heads=4, num_hidden_layers=2, multiple_of=2)
    model = phi.Phi(cfg).eval()
    x = ids(seq=10)
    full = model(x)
    cache = model.build_kv_cache(2)
    parts = [model(x[:, :6], cache, 0)] + [model(x[:, t : t + 1], cache, t) for t in range(6, 10)]
    assert torch.allclose(torch.cat(parts, 1), full, atol=1e-4)
    names = phi.Phi._huggingface_state_dict_map(2)
    assert set(names) == set(model.state_dict())


def test_mamba_parallel_sequential_and_step_agree():
    torch.manual_seed(0)
    cfg = mamba.MambaConfig(d_model=16, n_layers=2)
    model = mamba.Mamba(cfg).eval()
    x = torch.randn(2, 9, 16)
    parallel = model(x)
    cfg.pscan = False
    assert torch.allclose(parallel, model(x), atol=1e-5)
    caches = model.init_caches(2)
    steps = []
    for t in range(9):
        y, caches = model.step(x[:, t], caches)
        steps.append(y)
    assert torch.allclose(torch.stack(steps, 1), parallel, atol=1e-4)


@pytest.mark.parametrize("kind", ["lora", "dora"])
def test_adapters_replace_train_and_merge(kind):
    torch.manual_seed(0)
    cls, replace, mark, merge = {
        "lora": (LoRALinear, replace_with_lora, mark_lora_as_trainable, merge_lora),
        "dora": (DoRALinear, replace_with_dora, mark_dora_as_trainable, merge_dora),
    }[kind]
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    x = torch.randn(5, 8)
    before = net(x)
    replace(net, rank=4)
    assert isinstance(net[0], cls) and isinstance(net[2], cls)
    assert torch.allclose(net(x), before, atol=1e-5)  # B = 0: adapters start as no-ops
    mark(net)
    trainable = {n for n, p in net.named_parameters() if p.requires_grad}
    assert trainable and all("lora_" in n or "magnitude" in n for n in trainable)
    with torch.no_grad():
        for m in net.modules():
            if isinstance(m, cls):
                m.lora_B.normal_(std=0.1)
    adapted = net(x)
    assert not torch.allclose(adapted, before, atol=1e-4)
    merge(net)
    assert torch.allclose(net(x), adapted, atol=1e-5)
