"""Every model family against the reference package itself, when it is installed next to the
baseline (``baseline/_ref``): identical state-dict keys and shapes, and, loaded with the
reference's weights, identical outputs on the fp32 CPU path."""

import dataclasses
import importlib
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REFERENCE = ROOT / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REFERENCE / "ohara").is_dir(),
                                reason="reference package is not installed")

FAMILIES = {"llama": ("Config", "Llama"), "gpt": ("Config", "GPT"), "gemma": ("GemmaConfig", "Gemma"),
            "phi": ("PhiConfig", "Phi"), "retnet": ("Config", "RetNet"),
            "roformer": ("Config", "RoFormer"), "transformer": ("Config", "ModelingLM")}
SMALL = {"vocab": 128, "layers": 2, "width": 64, "ffn": 128, "heads": 4, "kv_heads": 2,
         "head_dim": 16, "context": 32}


@pytest.fixture(scope="module")
def reference_on_path():
    added = [str(ROOT / "baseline" / "stubs"), str(REFERENCE)]
    sys.path[:0] = added
    yield
    for entry in added:
        sys.path.remove(entry)


def _small(config_class) -> dict:
    """Toy sizes for whatever this family calls its fields."""
    chosen = {}
    for field in dataclasses.fields(config_class):
        name = field.name.lower()
        if "vocab" in name:
            chosen[field.name] = SMALL["vocab"]
        elif name in ("num_hidden_layers", "num_layers", "n_layers", "n_layer"):
            chosen[field.name] = SMALL["layers"]
        elif name in ("hidden_size", "d_model", "dim", "n_embd"):
            chosen[field.name] = SMALL["width"]
        elif name in ("intermediate_size", "hidden_dim"):
            chosen[field.name] = SMALL["ffn"]
        elif name in ("num_attention_heads", "num_heads", "n_head", "n_heads"):
            chosen[field.name] = SMALL["heads"]
        elif name in ("num_key_value_heads", "num_kv_heads"):
            chosen[field.name] = SMALL["kv_heads"]
        elif name == "head_dim":
            chosen[field.name] = SMALL["head_dim"]
        elif "seq" in name or name in ("block_size", "max_position_embeddings"):
            chosen[field.name] = SMALL["context"]
    return chosen


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_family_has_the_reference_layout_and_reproduces_its_outputs(reference_on_path, family):
    config_name, model_name = FAMILIES[family]
    theirs = importlib.import_module(f"ohara.models.{family}")
    ours = importlib.import_module(f"ohara_b200.models.{family}")
    sizes = _small(getattr(theirs, config_name))
    torch.manual_seed(0)
    reference = getattr(theirs, model_name)(getattr(theirs, config_name)(**sizes)).eval()
    torch.manual_seed(0)
    model = getattr(ours, model_name)(getattr(ours, config_name)(**sizes)).eval()
    want, have = reference.state_dict(), model.state_dict()
    assert list(want) == list(have)                  # same names, created in the same order ...
    assert all(tuple(want[k].shape) == tuple(have[k].shape) for k in want)
    for name in want:                                # ... so one seed gives the same initial model
        assert torch.equal(want[name], have[name]), name
    with torch.no_grad():
        for tensor in have.values():
            if tensor.is_floating_point():
                tensor.add_(1.0)                     # (make sure the load below does the work)
    model.load_state_dict(want)
    tokens = torch.randint(0, SMALL["vocab"], (2, 8))
    with torch.no_grad():
        a, b = reference(tokens), model(tokens)
    a, b = (a[0] if isinstance(a, tuple) else a), (b[0] if isinstance(b, tuple) else b)
    torch.testing.assert_close(b, a, rtol=1e-5, atol=2e-6)


def test_mamba_layers_and_their_recurrent_step_reproduce_the_reference(reference_on_path):
    theirs = importlib.import_module("ohara.models.mamba")
    ours = importlib.import_module("ohara_b200.models.mamba")
    torch.manual_seed(0)
    reference = theirs.Mamba(theirs.MambaConfig(d_model=64, n_layers=2)).eval()
    model = ours.Mamba(ours.MambaConfig(d_model=64, n_layers=2)).eval()
    model.load_state_dict(reference.state_dict())
    x = torch.randn(2, 8, 64)

    def stepwise(m):
        caches = [(None, torch.zeros(2, m.config.d_inner, m.config.d_conv - 1))
                  for _ in range(m.config.n_layers)]
        outputs = []
        for t in range(x.shape[1]):
            y, caches = m.step(x[:, t], caches)
            outputs.append(y)
        return torch.stack(outputs, 1)

    with torch.no_grad():
        torch.testing.assert_close(model(x), reference(x), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(stepwise(model), stepwise(reference), rtol=1e-5, atol=2e-6)
        torch.testing.assert_close(stepwise(model), model(x), rtol=1e-4, atol=2e-6)


def _twin_llamas(**extra):
    theirs = importlib.import_module("ohara.models.llama")
    ours = importlib.import_module("ohara_b200.models.llama")
    sizes = dict(vocab_size=96, max_sequence_length=32, hidden_size=48, intermediate_size=96,
                 num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, dropout=0.0,
                 weight_tying=False, **extra)
    torch.manual_seed(0)
    reference = theirs.Llama(theirs.Config(**sizes))
    model = ours.Llama(ours.Config(**sizes))
    model.load_state_dict(reference.state_dict())
    return reference, model


@pytest.mark.parametrize("builder", ["build_adamw", "build_muon_adamw", "build_adamh",
                                     "build_muonh_adamh"])
def test_optimizer_recipes_follow_the_reference_step_for_step(reference_on_path, builder):
    theirs = importlib.import_module("ohara.optimizer")
    ours = importlib.import_module("ohara_b200.optimizer")
    reference, model = _twin_llamas()
    kwargs = dict(learning_rate=3e-3, weight_decay=0.1) if builder == "build_adamw" else {}
    optimizers = (getattr(theirs, builder)(reference, **kwargs), getattr(ours, builder)(model, **kwargs))
    assert [(g.get("name"), g.get("kind"), len(g["params"])) for g in optimizers[0].param_groups] == \
        [(g.get("name"), g.get("kind"), len(g["params"])) for g in optimizers[1].param_groups]
    tokens = torch.randint(0, 96, (4, 17))
    for _ in range(3):
        for net, optimizer in zip((reference, model), optimizers):
            logits = net(tokens[:, :-1])
            loss = torch.nn.functional.cross_entropy(logits.flatten(0, 1), tokens[:, 1:].flatten())
            optimizer.zero_grad(set_to_none=True)
            loss.backward()
            optimizer.step()
    # (entries whose gradient is of the order of Adam's epsilon, behind the zero-initialised
    # output projections, differ by a fraction of a percent of one learning-rate-sized step
    # between formulations of the same update)
    for (name, want), have in zip(reference.state_dict().items(), model.state_dict().values()):
        torch.testing.assert_close(have, want, rtol=1e-4, atol=5e-5, msg=name)


@pytest.mark.parametrize("grouped", [False, True])
def test_mixture_of_experts_models_route_and_balance_like_the_reference(reference_on_path, grouped):
    reference, model = _twin_llamas(moe_num_experts=4, moe_experts_per_tok=2, moe_grouped=grouped,
                                    **({"moe_num_shared_experts": 1} if grouped else {}))
    with torch.no_grad():   # the routed output projections start at zero: give them values
        for name, p in reference.named_parameters():
            if name.endswith("w_down") or ".down.weight" in name:
                p.normal_(std=0.05)
    model.load_state_dict(reference.state_dict())
    theirs_moe = importlib.import_module("ohara.modules.moe")
    ours_moe = importlib.import_module("ohara_b200.modules.moe")
    tokens = torch.randint(0, 96, (3, 12))
    reference.train(), model.train()
    for step in range(3):
        with torch.no_grad():
            a, b = reference(tokens), model(tokens)
        # a token whose two best experts are tied to within rounding may be routed differently;
        # every other token must agree
        same = (a - b).abs().amax(-1) <= 2e-5
        assert (step > 0 or bool(same.all())) and float(same.float().mean()) >= 0.9
        theirs_moe.apply_qb_update(reference)
        ours_moe.apply_qb_update(model)
        for theirs_block, ours_block in zip(reference.layers, model.layers):
            torch.testing.assert_close(ours_block.ff.router_bias, theirs_block.ff.router_bias,
                                       rtol=1e-3, atol=1e-5)
    loads = ours_moe.expert_load(model), theirs_moe.expert_load(reference)
    assert loads[0].shape == loads[1].shape and int(loads[0].sum()) == int(loads[1].sum())
    assert float((loads[0] - loads[1]).abs().sum()) <= 0.1 * float(loads[1].sum())


def test_chat_rendering_and_sampling_agree_with_the_reference(reference_on_path):
    theirs_chat = importlib.import_module("ohara.chat")
    ours_chat = importlib.import_module("ohara_b200.chat")
    theirs_engine = importlib.import_module("ohara.chat_engine")
    ours_engine = importlib.import_module("ohara_b200.chat_engine")
    assert theirs_chat.CHAT_SPECIAL_TOKENS == ours_chat.CHAT_SPECIAL_TOKENS
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import chat_tokenizer

    tokenizer = chat_tokenizer()
    messages = [
        {"role": "system", "content": "be brief"}, {"role": "user", "content": "two plus two"},
        {"role": "assistant", "content": [{"type": "text", "text": "let me see "},
                                          {"type": "python", "text": "2+2"},
                                          {"type": "python_output", "text": "4"},
                                          {"type": "text", "text": "four"}]},
        {"role": "user", "content": "thanks"}, {"role": "assistant", "content": "welcome"}]
    for limit in (2048, 12):
        assert ours_chat.render_conversation(tokenizer, messages, max_tokens=limit) == \
            theirs_chat.render_conversation(tokenizer, messages, max_tokens=limit)
    assert ours_chat.render_for_completion(tokenizer, messages) == \
        theirs_chat.render_for_completion(tokenizer, messages)
    logits = torch.randn(3, 2, 50, generator=torch.Generator().manual_seed(0))   # (batch, seq, vocab)
    for settings in (dict(temperature=0.0), dict(temperature=0.8, top_k=5),
                     dict(temperature=1.2, top_p=0.7), dict(temperature=1.0, top_k=10, top_p=0.9)):
        picks = []
        for module in (theirs_engine, ours_engine):
            config = module.SamplingConfig(max_new_tokens=4, **settings)
            generator = torch.Generator().manual_seed(5)
            picks.append(module.sample_next_token(logits, config, generator))
        assert torch.equal(picks[0], picks[1]), settings


def test_planner_packer_and_token_files_are_interchangeable(reference_on_path, tmp_path):
    import dataclasses as dc

    theirs_scaling = importlib.import_module("ohara.scaling")
    ours_scaling = importlib.import_module("ohara_b200.scaling")
    for depth, budget in ((6, 1e15), (12, 3e17), (20, 1e19)):
        plans = [module.plan_scaling_run(depth=depth, flops_budget=budget, vocab_size=50304,
                                         sequence_length=1024, world_size=8)
                 for module in (theirs_scaling, ours_scaling)]
        assert dc.asdict(plans[0]) == dc.asdict(plans[1])

    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import chat_tokenizer

    tokenizer = chat_tokenizer()
    conversations = [{"messages": [
        {"role": "user", "content": " ".join(f"w{i * 7 + j}" for j in range(3 + i % 5))},
        {"role": "assistant", "content": " ".join(f"a{i + j}" for j in range(2 + i % 7))}]}
        for i in range(40)]
    packed = []
    for name in ("ohara.sft", "ohara_b200.sft"):
        dataset = importlib.import_module(name).ConversationDataset(
            conversations, tokenizer, max_length=32, seed=3, data_rank=1, data_world_size=2)
        rows = iter(dataset)
        packed.append([next(rows) for _ in range(6)])
    for (x_a, y_a), (x_b, y_b) in zip(*packed):
        assert torch.equal(x_a, x_b) and torch.equal(y_a, y_b)

    theirs_bin = importlib.import_module("ohara.tokenbin")
    ours_bin = importlib.import_module("ohara_b200.tokenbin")
    documents = [" ".join(f"t{(i * 13 + j) % 90}" for j in range(5 + i % 9)) for i in range(60)]
    written = {}
    for label, module in (("theirs", theirs_bin), ("ours", ours_bin)):
        path = tmp_path / f"{label}.bin"
        module.write_token_bin(documents, tokenizer, path, log=False)
        written[label] = path
    assert written["theirs"].read_bytes() == written["ours"].read_bytes()
    assert theirs_bin.read_token_bin_metadata(written["ours"]) == \
        ours_bin.read_token_bin_metadata(written["theirs"])
    blocks = []
    for module, path in ((theirs_bin, written["ours"]), (ours_bin, written["theirs"])):
        dataset = module.TokenBinDataset(path, max_length=16, shuffle=True, seed=7, infinite=False)
        blocks.append([tuple(t.tolist() for t in pair) for pair in dataset])
    assert blocks[0] == blocks[1] and len(blocks[0]) > 3


def test_trainer_and_generation_follow_the_reference(reference_on_path):
    from torch.utils.data import DataLoader, TensorDataset

    reference, model = _twin_llamas()
    tokens = torch.randint(0, 96, (16, 17), generator=torch.Generator().manual_seed(2))
    for package, net in (("ohara", reference), ("ohara_b200", model)):
        pkg = importlib.import_module(package)
        optimizer_module = importlib.import_module(f"{package}.optimizer")
        scheduler_module = importlib.import_module(f"{package}.lr_scheduler")
        engine = pkg.OharaEngine()
        net = engine.prepare(net)
        optimizer = optimizer_module.build_adamw(net, learning_rate=1e-2, weight_decay=0.1)
        (optimizer,) = engine.prepare_optimizers(optimizer)
        loader = engine.prepare_dataloaders(
            DataLoader(TensorDataset(tokens[:, :-1], tokens[:, 1:]), batch_size=4))
        trainer = pkg.Trainer(engine, net, optimizer, loader, loader,
                              scheduler_module.Scheduler(1e-2), micro_batch=2, max_iters=4,
                              eval_iters=0, save_ckpt_iters=0, print_every=10**9)
        trainer.train()
    for (name, want), have in zip(reference.state_dict().items(), model.state_dict().values()):
        torch.testing.assert_close(have, want, rtol=1e-4, atol=5e-5, msg=name)

    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import chat_tokenizer

    tokenizer = chat_tokenizer()
    reference, model = _twin_llamas()
    outputs = []
    for package, net in (("ohara.chat_engine", reference), ("ohara_b200.chat_engine", model)):
        module = importlib.import_module(package)
        chat = module.ChatEngine(net.eval(), tokenizer, device="cpu")
        config = module.SamplingConfig(temperature=0.9, top_k=20, top_p=0.95, max_new_tokens=10)
        messages = [{"role": "user", "content": "w1 w2 w3"}]
        outputs.append((chat.render_prompt(messages), chat.generate(messages, config, seed=11),
                        chat.generate(messages, module.SamplingConfig(temperature=0.0,
                                                                      max_new_tokens=8))))
    assert outputs[0] == outputs[1] and outputs[0][1] and outputs[0][2]


def test_recurrent_unit_follows_the_paper_and_can_reproduce_the_reference(reference_on_path):
    """The reference's RG-LRU scans over the width (its unit has no memory); this package's scans
    over time, and a switch gives the reference's function for checkpoints trained with it."""
    theirs = importlib.import_module("ohara.modules.linear_rnn")
    ours = importlib.import_module("ohara_b200.modules.linear_rnn")
    torch.manual_seed(0)
    reference, unit = theirs.Hawk(dim=16), ours.Hawk(dim=16)
    unit.load_state_dict(reference.state_dict())
    x = torch.randn(2, 9, 16)
    assert not torch.allclose(unit(x), reference(x), atol=1e-4)
    unit.linear_rnn.scan_over_width = True
    torch.testing.assert_close(unit(x), reference(x), rtol=1e-5, atol=1e-6)


def test_schedules_losses_adaptors_positions_and_caches_match(reference_on_path):
    def pair(module):
        return (importlib.import_module("ohara." + module),
                importlib.import_module("ohara_b200." + module))

    torch.manual_seed(0)
    theirs, ours = pair("lr_scheduler")
    a, b = theirs.CosineScheduler(3e-4, 3e-5, 10, 100), ours.CosineScheduler(3e-4, 3e-5, 10, 100)
    assert all(a(i) == b(i) for i in range(130))
    theirs, ours = pair("scaling")
    for name, arguments, steps in (("WarmupStableDecayScheduler", (0.02, 200), 201),
                                   ("MuonMomentumScheduler", (300,), 301),
                                   ("CosineWeightDecayScheduler", (0.1, 100), 101)):
        a, b = getattr(theirs, name)(*arguments), getattr(ours, name)(*arguments)
        assert all(a(i) == b(i) for i in range(steps)), name

    theirs, ours = pair("dpo")
    logps = [torch.randn(6) for _ in range(4)]
    for name in ("dpo_loss_from_logps", "ipo_loss_from_logps", "cdpo_loss_from_logps"):
        for want, got in zip(getattr(theirs, name)(*logps, 0.3), getattr(ours, name)(*logps, 0.3)):
            torch.testing.assert_close(got, want)
    logits, labels = torch.randn(2, 7, 11), torch.randint(0, 11, (2, 7))
    labels[0, :3] = theirs.IGNORE_INDEX
    torch.testing.assert_close(ours.sequence_logps(logits, labels),
                               theirs.sequence_logps(logits, labels))

    theirs, ours = pair("swa")
    q, k, v = (torch.randn(2, 16, 8) for _ in range(3))
    torch.testing.assert_close(ours.sliding_window_attention_with_mask(q, k, v, 4),
                               theirs.sliding_window_attention_with_mask(q, k, v, 4))

    x = torch.randn(3, 16)
    for module, name in (("adaptor.lora", "LoRALinear"), ("adaptor.dora", "DoRALinear")):
        theirs, ours = pair(module)
        a, b = (getattr(m, name)(16, 8, rank=4, lora_alpha=2) for m in (theirs, ours))
        with torch.no_grad():
            for parameter in a.parameters():
                parameter.add_(torch.randn_like(parameter) * 0.1)
        b.load_state_dict(a.state_dict())
        torch.testing.assert_close(b(x), a(x))

    theirs, ours = pair("embeddings_pos.alibi")
    assert torch.equal(theirs.get_alibi_mask(8, 4), ours.get_alibi_mask(8, 4))
    theirs, ours = pair("embeddings_pos.xpos")
    def tensors(value):
        if torch.is_tensor(value):
            return [value]
        return [t for item in value for t in tensors(item)]

    for recurrent in (False, True):
        want = tensors(theirs.XPos(16, 4)(6, recurrent=recurrent))
        got = tensors(ours.XPos(16, 4)(6, recurrent=recurrent))
        assert len(want) == len(got) > 0
        for a, b in zip(want, got):
            torch.testing.assert_close(b, a)

    theirs, ours = pair("modules.kv_cache")
    for int8 in (False, True):
        a, b = (m.KVCache((2, 16, 2, 8), max_seq_length=16, int8=int8) for m in (theirs, ours))
        position = 0
        for steps in (5, 1, 1):
            keys, values = torch.randn(2, steps, 2, 8), torch.randn(2, steps, 2, 8)
            for want, got in zip(a.forward(keys, values, position), b.forward(keys, values, position)):
                torch.testing.assert_close(got, want)
            position += steps


def test_streaming_text_dataset_cuts_the_same_blocks(reference_on_path, monkeypatch):
    """Both packages read a (stubbed) ``datasets`` stream: same calls into the library, same
    token blocks with and without shuffling, per-rank sharding and a resume offset."""
    import random
    import types

    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import WordTokenizer

    documents = [{"text": " ".join(f"w{(i * 7 + j) % 50}" for j in range(5 + i % 11))}
                 for i in range(60)]

    class Stream:
        def __init__(self, rows):
            self.rows = rows

        def __iter__(self):
            return iter(self.rows)

        def shuffle(self, seed=None, buffer_size=None):
            rows = list(self.rows)
            random.Random(seed).shuffle(rows)
            return Stream(rows)

    calls = []

    def load_dataset(*args, **kwargs):
        calls.append((args, tuple(sorted(kwargs.items()))))
        return Stream(documents)

    stub = types.ModuleType("datasets")
    stub.load_dataset, stub.load_from_disk = load_dataset, (lambda *a, **k: None)
    monkeypatch.setitem(sys.modules, "datasets", stub)
    blocks = {}
    for package in ("ohara", "ohara_b200"):
        module = importlib.import_module(package + ".dataset")
        monkeypatch.setattr(module, "load_dataset", load_dataset, raising=False)
        for shuffle in (False, True):
            for rank, world, start in ((None, None, 2), (1, 2, 0)):
                dataset = module.StreamingTextDataset(
                    "some/corpus", WordTokenizer(), split="train", max_length=16, shuffle=shuffle,
                    seed=3, data_rank=rank, data_world_size=world, start_block=start)
                rows = iter(dataset)
                blocks[(package, shuffle, rank)] = [tuple(t.tolist() for t in next(rows))
                                                    for _ in range(6)]
    for (package, shuffle, rank), rows in blocks.items():
        if package == "ohara":
            assert rows == blocks[("ohara_b200", shuffle, rank)], (shuffle, rank)
    assert calls[: len(calls) // 2] == calls[len(calls) // 2:]
