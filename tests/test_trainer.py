"""Trainer behaviour: metrics, schedules, accumulation equivalence, checkpoints, guards."""

import math
from pathlib import Path

import pytest
import torch
import torch.nn as nn
from torch.utils.data import DataLoader, Dataset, TensorDataset

from ohara_b200.lr_scheduler import CosineScheduler, Scheduler
from ohara_b200.models.llama import Config, Llama
from ohara_b200.optimizer import build_adamw, build_muon_adamw
from ohara_b200.runtime import EngineConfig, OharaEngine, PrecisionConfig, PrecisionMode
from ohara_b200.trainer import Trainer


class EchoDataset(Dataset):
    """inputs == targets so a model that echoes its input scores perfectly."""

    def __init__(self, n=16, seq=8, vocab=11):
        gen = torch.Generator().manual_seed(0)
        self.rows = torch.randint(0, vocab, (n, seq), generator=gen)

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i], self.rows[i].clone()


class EchoModel(nn.Module):
    """Logits are one-hot(input) * scale: loss is known in closed form."""

    def __init__(self, vocab=11, scale=5.0):
        super().__init__()
        self.vocab = vocab
        self.scale = nn.Parameter(torch.tensor(scale))

    def forward(self, x):
        return torch.nn.functional.one_hot(x, self.vocab).float() * self.scale


def make_trainer(tmp_path, model=None, dataset=None, **kw):
    engine = OharaEngine()
    engine.launch()
    model = engine.prepare(model or EchoModel())
    opt = torch.optim.SGD(model.parameters(), lr=0.0)
    dl = DataLoader(dataset or EchoDataset(), batch_size=4)
    args = dict(micro_batch=1, max_iters=2, eval_iters=0, save_ckpt_iters=0,
                checkpoint_path=tmp_path / "ckpt" / "model.pt")
    args.update(kw)
    return Trainer(engine, model, opt, dl, dl, Scheduler(0.0), **args), engine


def test_constructor_validation(tmp_path):
    for bad in (dict(micro_batch=0), dict(max_iters=0), dict(eval_iters=-1),
                dict(eval_val_batches=0), dict(iter_loss_window=0),
                dict(token_bytes=torch.zeros(2, 2))):
        with pytest.raises(ValueError):
            make_trainer(tmp_path, **bad)


def test_evaluate_metrics_closed_form(tmp_path):
    trainer, _ = make_trainer(tmp_path)
    metrics = trainer.evaluate(trainer.val_dataloader, 2)
    expected = math.log(math.exp(5.0) + 10) - 5.0
    assert math.isclose(metrics["loss"], expected, rel_tol=1e-5)
    assert math.isclose(metrics["ppl"], math.exp(expected), rel_tol=1e-5)
    assert math.isclose(metrics["bits_per_token"], expected / math.log(2), rel_tol=1e-5)
    assert metrics["accuracy"] == 1.0
    assert metrics["tokens"] == 2 * 4 * 8


def test_bits_per_byte_uses_token_bytes(tmp_path):
    token_bytes = torch.arange(11, dtype=torch.int32)  # token 0 has zero bytes and is skipped
    trainer, _ = make_trainer(tmp_path, token_bytes=token_bytes)
    metrics = trainer.evaluate(trainer.val_dataloader, 1)
    rows = EchoDataset().rows[:4].reshape(-1)
    counted = rows[rows > 0]
    per_token = math.log(math.exp(5.0) + 10) - 5.0
    expected = per_token * len(counted) / (math.log(2) * float(counted.sum()))
    assert math.isclose(metrics["bpb"], expected, rel_tol=1e-5)
    assert metrics["bytes"] == float(counted.sum())


def test_evaluation_does_not_advance_training_iterator_and_caches_validation(tmp_path):
    trainer, _ = make_trainer(tmp_path)
    first = next(trainer.train_dataloader)
    trainer.train_dataloader.close()
    trainer.evaluate(trainer.train_dataloader, 3)
    trainer.evaluate(trainer.val_dataloader, 2)
    assert len(trainer._validation_batches) == 2
    again = next(trainer.train_dataloader)
    assert torch.equal(first[0], again[0])
    cached = trainer._validation_batches
    trainer.evaluate(trainer.val_dataloader, 2)
    assert trainer._validation_batches is cached


def test_lr_scale_and_muon_only_hparams(tmp_path):
    torch.manual_seed(0)
    cfg = Config(vocab_size=11, max_sequence_length=8, hidden_size=16, intermediate_size=24,
                 num_attention_heads=2, num_hidden_layers=1, dropout=0.0)
    engine = OharaEngine()
    model = engine.prepare(Llama(cfg))
    opt = build_muon_adamw(model)
    dl = DataLoader(EchoDataset(), batch_size=4)
    trainer = Trainer(engine, model, opt, dl, dl, lambda it: 0.01, micro_batch=1, max_iters=1,
                      eval_iters=0, save_ckpt_iters=0,
                      get_optimizer_hparams=lambda it: {"momentum": 0.5, "weight_decay": 0.3})
    trainer.train()
    for group in opt.param_groups:
        assert math.isclose(group["lr"], 0.01 * group["lr_scale"])
        if group["kind"] == "muon":
            assert group["momentum"] == 0.5 and group["weight_decay"] == 0.3
        else:
            assert group["weight_decay"] != 0.3
    bad = Trainer(engine, model, opt, dl, dl, lambda it: 0.01, micro_batch=1, max_iters=1,
                  eval_iters=0, save_ckpt_iters=0, get_optimizer_hparams=lambda it: {"beta": 1.0})
    with pytest.raises(ValueError):
        bad.train()


def test_invalid_lr_and_empty_batches_raise(tmp_path):
    trainer, _ = make_trainer(tmp_path)
    trainer.get_lr = lambda it: float("nan")
    with pytest.raises(RuntimeError):
        trainer.train()

    class AllIgnored(Dataset):
        def __len__(self):
            return 4

        def __getitem__(self, i):
            return torch.zeros(8, dtype=torch.long), torch.full((8,), -1)

    trainer, _ = make_trainer(tmp_path, dataset=AllIgnored())
    with pytest.raises(RuntimeError):
        trainer.train()


def test_checkpoint_round_trip_and_no_temp_files(tmp_path):
    trainer, engine = make_trainer(tmp_path, save_ckpt_iters=2)
    trainer.train()
    ckpt = tmp_path / "ckpt" / "model.pt"
    assert ckpt.exists()
    assert [p.name for p in ckpt.parent.iterdir()] == ["model.pt"]
    payload = engine.load(ckpt)
    for key in ("model", "optimizer", "idx", "lr", "train_step_loss",
                "gradient_accumulation_steps", "train_batches_consumed", "torch_rng_state"):
        assert key in payload
    assert payload["idx"] == 2 and payload["train_batches_consumed"] == 2
    fresh = EchoModel(scale=1.0)
    engine.load(ckpt, {"model": fresh})
    assert float(fresh.scale) == 5.0


def test_grad_accumulation_equals_single_batch_with_ignored_tokens():
    torch.manual_seed(0)
    cfg = Config(vocab_size=23, max_sequence_length=8, hidden_size=16, intermediate_size=24,
                 num_attention_heads=2, num_hidden_layers=1, dropout=0.0)
    ids = torch.randint(0, 23, (8, 9))
    x, y = ids[:, :-1], ids[:, 1:].clone()
    y[0, :6] = -1
    y[5, 2:] = -1

    def run(batch_size, micro_batch):
        torch.manual_seed(1)
        engine = OharaEngine()
        model = engine.prepare(Llama(cfg))
        opt = build_adamw(model, learning_rate=1e-2, weight_decay=0.0)
        dl = DataLoader(TensorDataset(x, y), batch_size=batch_size)
        trainer = Trainer(engine, model, opt, dl, dl, Scheduler(1e-2), micro_batch=micro_batch,
                          max_iters=1, eval_iters=0, save_ckpt_iters=0)
        trainer.train()
        return [p.detach().clone() for p in model.parameters()], trainer.last_step_loss

    whole, loss_whole = run(8, 1)
    pieces, loss_pieces = run(2, 4)
    assert math.isclose(loss_whole, loss_pieces, rel_tol=1e-5)
    for a, b in zip(whole, pieces):
        assert torch.allclose(a, b, atol=1e-5)


def test_end_to_end_loss_halves():
    torch.manual_seed(0)
    cfg = Config(vocab_size=17, max_sequence_length=16, hidden_size=32, intermediate_size=48,
                 num_attention_heads=2, num_hidden_layers=2, dropout=0.0)
    pattern = (torch.arange(16)[:, None] + torch.arange(17)[None, :]) % 17
    ds = TensorDataset(pattern[:, :-1], pattern[:, 1:])
    engine = OharaEngine()
    model = engine.prepare(Llama(cfg))
    opt = build_muon_adamw(model)
    dl = DataLoader(ds, batch_size=8)
    trainer = Trainer(engine, model, opt, dl, dl, CosineScheduler(0.02, 0.002, 2, 12),
                      micro_batch=1, max_iters=12, eval_iters=0, save_ckpt_iters=0)
    first = trainer.evaluate(trainer.val_dataloader, 2)["loss"]
    trainer.train()
    assert trainer.evaluate(trainer.val_dataloader, 2)["loss"] < 0.5 * first


def test_bf16_true_casts_module():
    engine = OharaEngine(EngineConfig(precision=PrecisionConfig(PrecisionMode.BF16_TRUE)))
    model = engine.prepare(nn.Linear(4, 4))
    assert model.weight.dtype == torch.bfloat16


def test_cosine_scheduler_edges():
    sched = CosineScheduler(learning_rate=1.0, min_lr=0.1, warmup_iters=10, max_iters=110)
    assert sched(0) == 0.0 and sched(5) == 0.5
    assert math.isclose(sched(10), 1.0) and math.isclose(sched(110), 0.1)
    assert math.isclose(sched(60), 0.55) and sched(500) == 0.1
    for bad in (dict(learning_rate=-1), dict(min_lr=2.0), dict(warmup_iters=-1),
                dict(max_iters=0), dict(warmup_iters=200, max_iters=100)):
        with pytest.raises(ValueError):
            CosineScheduler(**{**dict(learning_rate=1.0, min_lr=0.1, warmup_iters=10, max_iters=110), **bad})
    with pytest.raises(ValueError):
        sched(-1)


def test_profile_sections_report_every_phase_of_the_step(tmp_path):
    trainer, _ = make_trainer(tmp_path, profile_sections=True, grad_clip_norm=1.0, max_iters=2)
    trainer.train()
    times = trainer.section_times()
    assert set(times) == {"train.forward_backward", "train.clip", "train.optimizer"}
    assert all(entry["calls"] == 2 and entry["ms"] >= 0.0 for entry in times.values())
    assert trainer.section_times() == {}  # reset by the previous call
    plain, _ = make_trainer(tmp_path)
    assert plain.section_times() == {}
