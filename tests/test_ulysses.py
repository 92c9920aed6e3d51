"""Ulysses-style context parallelism (all-to-all between sequence shards and head shards) on
gloo ranks: the exchanges are inverses of each other and a model trained with its sequences cut
over the ranks follows single-process training."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _run(script: str, world: int, tmp_path, port: int) -> str:
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    from helpers import run_ranks

    code, stdout, stderr = run_ranks(path, world, port=port + os.getpid() % 150, env=env)
    assert code == 0, stdout[-3000:] + stderr[-3000:]
    return stdout


def test_exchanges_are_inverses_and_attention_matches_the_whole_sequence(tmp_path):
    out = _run(
        """
        import torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.parallel.cp import shard_sequence
        from ohara_b200.parallel.ulysses import (UlyssesWorkspace, heads_to_sequence,
                                                 sequence_to_heads, ulysses_attention)
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        workspace = UlyssesWorkspace(dist.group.WORLD)
        torch.manual_seed(0)
        B, T, H, Hk, D = 2, 8 * world, 4, 1, 8          # one key/value head: repeated over the ranks
        q, k, v = torch.randn(B, T, H, D), torch.randn(B, T, Hk, D), torch.randn(B, T, Hk, D)
        mine = [shard_sequence(t, rank, world).clone().requires_grad_() for t in (q, k, v)]
        there = sequence_to_heads(mine[0], workspace)
        assert there.shape == (B, T, H // world, D)
        assert torch.equal(heads_to_sequence(there, workspace), mine[0])
        out = ulysses_attention(*mine, workspace)
        full = [t.clone().requires_grad_() for t in (q, k, v)]
        want = ops.attention(*full, causal=True)
        assert torch.allclose(out, shard_sequence(want, rank, world), atol=1e-5)
        weight = torch.randn(B, T, H, D)
        (out * shard_sequence(weight, rank, world)).sum().backward()
        (want * weight).sum().backward()
        for got, ref in zip(mine, full):
            assert torch.allclose(got.grad, shard_sequence(ref.grad, rank, world), atol=1e-5)
        if rank == 0:
            print("ULYSSES_OP_OK")
        dist.destroy_process_group()
        """, 2, tmp_path, 30500)
    assert "ULYSSES_OP_OK" in out


@pytest.mark.parametrize("world,cp", [(4, 2)])
def test_training_with_sequences_cut_over_the_ranks_matches_single_process(tmp_path, world, cp):
    out = _run(
        f"""
        import torch, torch.distributed as dist
        from torch.utils.data import DataLoader, TensorDataset
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, ParallelConfig, StrategyType
        from ohara_b200.optimizer import build_adamw
        from ohara_b200.trainer import Trainer
        from ohara_b200.lr_scheduler import Scheduler

        torch.manual_seed(0)
        cfg = Config(vocab_size=31, max_sequence_length=16, hidden_size=16, intermediate_size=24,
                     num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, dropout=0.0)
        ids = torch.randint(0, 31, (8, 17))
        dataset = TensorDataset(ids[:, :-1], ids[:, 1:])
        state = {{k: v.clone() for k, v in Llama(cfg).state_dict().items()}}
        solo = Llama(cfg); solo.load_state_dict(state)
        ref_opt = build_adamw(solo, learning_rate=0.02, weight_decay=0.1)
        for _ in range(3):
            loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
            loss.backward(); ref_opt.step(); ref_opt.zero_grad()

        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP,
                                          parallel=ParallelConfig(cp={cp}),
                                          context_parallel_mode="ulysses"))
        model = Llama(cfg); model.load_state_dict(state)
        model = engine.prepare(model)
        (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
        dp = engine.data_parallel_world_size
        assert dp == {world} // {cp}
        loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=8 // dp))
        trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                          max_iters=3, eval_iters=0, save_ckpt_iters=0)
        trainer.train()
        full = engine.full_state_dict(model)
        for name, value in solo.state_dict().items():
            assert torch.allclose(full[name], value, atol=3e-5), (name, (full[name] - value).abs().max())
        if dist.get_rank() == 0:
            print("ULYSSES_TRAIN_OK")
        engine.close()
        """, world, tmp_path, 30700)
    assert "ULYSSES_TRAIN_OK" in out
