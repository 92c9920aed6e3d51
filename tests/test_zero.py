"""Sharded optimizer: layout invariants (single process) and equivalence with unsharded training
on two gloo ranks."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import torch

from helpers import launch_ranks
from ohara_b200.models.llama import Config, Llama
from ohara_b200.optimizer import build_adamw, build_muon_adamw
from ohara_b200.parallel.zero import ShardedOptimizer

ROOT = Path(__file__).resolve().parent.parent


def small():
    return Llama(Config(vocab_size=61, max_sequence_length=16, hidden_size=32, intermediate_size=48,
                        num_attention_heads=2, num_hidden_layers=2, dropout=0.0))


def test_single_rank_sharded_optimizer_matches_plain():
    torch.manual_seed(0)
    a, b = small(), small()
    b.load_state_dict(a.state_dict())
    plain = build_muon_adamw(a)
    sharded = ShardedOptimizer(build_muon_adamw(b))
    covered = sum(piece.length for piece in sharded.all_pieces)
    assert covered == sum(p.numel() for p in b.parameters())
    ids = torch.randint(0, 61, (4, 13))
    for _ in range(3):
        for model, opt in ((a, plain), (b, sharded)):
            loss = model.loss_sum(ids[:, :-1], ids[:, 1:]) / 48
            loss.backward()
            opt.step()
            opt.zero_grad()
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert torch.allclose(pa, pb, atol=1e-6)
    norm = sharded.clip_grad_norm_(b, 1.0)
    assert float(norm) == 0.0  # no gradients pending


def _run(script, world, tmp_path):
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, world, port=29000 + os.getpid() % 500, env=env, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    return proc.stdout


def test_two_rank_sharded_training_matches_single_process(tmp_path):
    out = _run(
        """
        import torch, torch.distributed as dist
        from torch.utils.data import DataLoader, TensorDataset
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, StrategyType
        from ohara_b200.optimizer import build_muon_adamw
        from ohara_b200.trainer import Trainer
        from ohara_b200.lr_scheduler import Scheduler
        torch.manual_seed(0)
        cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
                     num_attention_heads=2, num_hidden_layers=2, dropout=0.0)
        ids = torch.randint(0, 31, (8, 9))
        ds = TensorDataset(ids[:, :-1], ids[:, 1:])
        base = Llama(cfg)
        state = {k: v.clone() for k, v in base.state_dict().items()}
        solo = Llama(cfg); solo.load_state_dict(state)
        opt = build_muon_adamw(solo)
        for _ in range(3):
            loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
            loss.backward(); opt.step(); opt.zero_grad()
        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP))
        model = Llama(cfg); model.load_state_dict(state)
        model = engine.prepare(model)
        (sharded,) = engine.prepare_optimizers(build_muon_adamw(model))
        assert type(sharded).__name__ == "ShardedOptimizer" and sharded.world == 2
        dl = engine.prepare_dataloaders(DataLoader(ds, batch_size=4))
        trainer = Trainer(engine, model, sharded, dl, dl, Scheduler(0.02), micro_batch=1,
                          max_iters=3, eval_iters=0, save_ckpt_iters=3,
                          checkpoint_path="%s/ck.pt")
        trainer.train()
        for a, b in zip(solo.parameters(), model.parameters()):
            assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()
        # state dict round trip at the same world size
        blob = sharded.state_dict()
        sharded.load_state_dict(blob)
        full = engine.full_state_dict(model)
        for key, value in solo.state_dict().items():
            assert torch.allclose(full[key], value, atol=2e-5), key
        if dist.get_rank() == 0:
            print("ZERO_OK")
        engine.close()
        """ % tmp_path,
        2, tmp_path,
    )
    assert "ZERO_OK" in out


def _assert_state_equal(mine, theirs, atol=1e-6):
    assert set(mine["state"]) == set(theirs["state"])
    for idx, entry in theirs["state"].items():
        for key, value in entry.items():
            got = mine["state"][idx][key]
            if isinstance(value, torch.Tensor):
                assert got.shape == value.shape, (idx, key, got.shape, value.shape)
                assert torch.allclose(got.float(), value.float(), atol=atol), (idx, key)
            else:
                assert got == value, (idx, key)
    for a, b in zip(mine["param_groups"], theirs["param_groups"]):
        assert a["params"] == b["params"] and a["lr"] == b["lr"] and a.get("kind") == b.get("kind")


def test_full_state_dict_has_the_unsharded_optimizers_format():
    torch.manual_seed(0)
    a, b = small(), small()
    b.load_state_dict(a.state_dict())
    plain = build_muon_adamw(a)
    sharded = ShardedOptimizer(build_muon_adamw(b))
    ids = torch.randint(0, 61, (4, 13))
    for _ in range(2):
        for model, opt in ((a, plain), (b, sharded)):
            (model.loss_sum(ids[:, :-1], ids[:, 1:]) / 48).backward()
            opt.step()
            opt.zero_grad()
    _assert_state_equal(sharded.full_state_dict(), plain.state_dict())
    # and the other direction: a plain optimizer's state continues inside a sharded one
    c = small()
    c.load_state_dict(a.state_dict())
    resumed = ShardedOptimizer(build_muon_adamw(c))
    resumed.load_state_dict(plain.state_dict())
    for model, opt in ((a, plain), (c, resumed)):
        (model.loss_sum(ids[:, :-1], ids[:, 1:]) / 48).backward()
        opt.step()
        opt.zero_grad()
    for pa, pc in zip(a.parameters(), c.parameters()):
        assert torch.allclose(pa, pc, atol=1e-6)


def test_checkpoint_of_two_ranks_resumes_on_one_and_on_three(tmp_path):
    """Train 2 steps on 2 ranks, save, then continue the third step at world sizes 1 and 3; all
    must land on the parameters of an uninterrupted single-process run."""
    common = """
        import torch, torch.distributed as dist
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.optimizer import build_muon_adamw
        from ohara_b200.parallel.zero import ShardedOptimizer
        torch.manual_seed(0)
        cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
                     num_attention_heads=2, num_hidden_layers=2, dropout=0.0)
        ids = torch.randint(0, 31, (12, 9))
        base = Llama(cfg)
        state = {k: v.clone() for k, v in base.state_dict().items()}
        def step(model, opt, rows):
            loss = model.loss_sum(ids[rows, :-1], ids[rows, 1:]) / ids[:, 1:].numel()
            loss.backward(); opt.step(); opt.zero_grad()
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        rows = slice(rank * 12 // world, (rank + 1) * 12 // world)
        path = "%s/reshard.pt"
    """ % tmp_path
    _run(common + """
        model = Llama(cfg); model.load_state_dict(state)
        opt = ShardedOptimizer(build_muon_adamw(model))
        assert opt.world == 2
        # the sharded optimizer averages over ranks; the loss is already divided by all tokens
        for p in model.parameters(): p.register_hook(lambda g: g * world)
        for _ in range(2):
            step(model, opt, rows)
        opt.sync_master_weights()
        blob = {"model": model.state_dict(), "optimizer": opt.state_dict()}
        if rank == 0:
            torch.save(blob, path)
        dist.barrier()
    """, 2, tmp_path)
    for world in (1, 3):
        out = _run(common + """
        solo = Llama(cfg); solo.load_state_dict(state)
        plain = build_muon_adamw(solo)
        for _ in range(3):
            step(solo, plain, slice(0, 12))
        blob = torch.load(path, weights_only=False)
        assert blob["optimizer"]["world_size"] == 2
        model = Llama(cfg); model.load_state_dict(blob["model"])
        opt = ShardedOptimizer(build_muon_adamw(model))
        opt.load_state_dict(blob["optimizer"])
        for p in model.parameters(): p.register_hook(lambda g: g * world)
        step(model, opt, rows)
        opt.sync_master_weights()
        for a, b in zip(solo.parameters(), model.parameters()):
            assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()
        if rank == 0:
            print("RESHARD_OK", world)
        """, world, tmp_path)
        assert f"RESHARD_OK {world}" in out
