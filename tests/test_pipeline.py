"""Pipeline schedules on gloo ranks: gradients and loss of a 3-stage pipeline must equal those of
the unsplit model on the whole batch, for both schedules."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from helpers import launch_ranks
import torch.nn as nn

from ohara_b200.parallel.pipeline import split_sequential

ROOT = Path(__file__).resolve().parent.parent


def test_split_sequential_is_contiguous_and_balanced():
    layers = [nn.Linear(2, 2) for _ in range(7)]
    parts = [split_sequential(layers, 3, r) for r in range(3)]
    assert [len(p) for p in parts] == [3, 2, 2]
    assert [m for p in parts for m in p] == layers
    with pytest.raises(ValueError):
        split_sequential(layers[:2], 3, 0)


@pytest.mark.parametrize("schedule", ["1f1b", "gpipe"])
def test_three_stage_pipeline_matches_the_unsplit_model(tmp_path, schedule):
    script = """
        import torch, torch.nn as nn, torch.distributed as dist
        from ohara_b200.parallel.pipeline import PipelineRunner, split_sequential
        from ohara_b200.runtime.enums import PipelineScheduleType
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        torch.manual_seed(0)
        layers = []
        for _ in range(6):
            layers += [nn.Linear(16, 16), nn.Tanh()]
        layers.append(nn.Linear(16, 4))
        full = nn.Sequential(*layers)
        x = torch.randn(10, 16)
        y = torch.randn(10, 4)
        loss_fn = lambda out, target: ((out - target) ** 2).mean()
        micro = 5
        xs, ys = x.chunk(micro), y.chunk(micro)
        reference = sum(loss_fn(full(a), b) for a, b in zip(xs, ys)) / micro
        reference.backward()
        expected = {id(p): p.grad.clone() for p in full.parameters()}
        for p in full.parameters():
            p.grad = None
        stage = split_sequential(layers, world, rank)
        runner = PipelineRunner(stage, loss_fn if rank == world - 1 else None,
                                schedule=PipelineScheduleType("%s"),
                                activation_shape=(2, 16), device="cpu")
        loss = runner.step(xs if rank == 0 else None, ys if rank == world - 1 else None, micro)
        for p in stage.parameters():
            assert torch.allclose(p.grad, expected[id(p)], atol=1e-6), (rank, (p.grad - expected[id(p)]).abs().max())
        if rank == world - 1:
            assert torch.allclose(loss, reference.detach(), atol=1e-6)
            print("PIPELINE_OK")
        dist.barrier()
    """ % schedule
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, 3, port=30600 + os.getpid() % 300, env=env, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "PIPELINE_OK" in proc.stdout


def test_llama_stage_bounds_cover_all_layers():
    from ohara_b200.parallel.pipeline import stage_bounds

    for layers, world in [(12, 4), (7, 3), (5, 5)]:
        spans = [stage_bounds(layers, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == layers
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        stage_bounds(2, 3, 0)


def test_llama_stage_rejects_tied_embeddings():
    from ohara_b200.models.llama import Config, Llama
    from ohara_b200.parallel.pipeline import LlamaStage

    cfg = Config(vocab_size=64, max_sequence_length=16, hidden_size=32, intermediate_size=64,
                 num_attention_heads=2, num_hidden_layers=2, dropout=0.0, weight_tying=True)
    with pytest.raises(ValueError):
        LlamaStage(Llama(cfg), 2, 0)


def test_llama_split_in_three_stages_matches_the_whole_model(tmp_path):
    """A 5-layer Llama as three pipeline stages (1F1B, 4 micro-batches) on gloo ranks: loss and the
    gradients of every stage's parameters equal those of the unsplit model."""
    script = """
        import torch, torch.distributed as dist
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.parallel.pipeline import LlamaStage, PipelineRunner
        from ohara_b200.runtime.enums import PipelineScheduleType
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        cfg = Config(vocab_size=96, max_sequence_length=24, hidden_size=32, intermediate_size=64,
                     num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=5, dropout=0.0,
                     weight_tying=False)
        torch.manual_seed(0)
        full = Llama(cfg).enable_activation_checkpointing()   # stages recompute their blocks too
        ids = torch.randint(0, 96, (8, 25))
        x, y = ids[:, :-1], ids[:, 1:]
        micro = 4
        xs, ys = x.chunk(micro), y.chunk(micro)
        stage = LlamaStage(full, world, rank)
        assert stage.activation_checkpointing
        reference = sum(stage.loss(full(a), b) for a, b in zip(xs, ys)) / micro
        reference.backward()
        expected = {name: p.grad.clone() for name, p in full.named_parameters()}
        full.zero_grad(set_to_none=True)
        owned = sum(p.numel() for p in stage.parameters())
        assert owned < sum(p.numel() for p in full.parameters())
        runner = PipelineRunner(stage, stage.loss if rank == world - 1 else None,
                                schedule=PipelineScheduleType.ONE_FWD_ONE_BWD,
                                activation_shape=(2, 24, 32), device="cpu")
        loss = runner.step(xs if rank == 0 else None, ys if rank == world - 1 else None, micro)
        names = {id(p): name for name, p in full.named_parameters()}
        checked = 0
        for p in stage.parameters():
            want = expected[names[id(p)]]
            assert torch.allclose(p.grad, want, atol=1e-5), (rank, names[id(p)])
            checked += 1
        assert checked > 0
        if rank == world - 1:
            assert torch.allclose(loss, reference.detach(), atol=1e-5)
            print("LLAMA_PIPELINE_OK")
        dist.barrier()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, 3, port=30950 + os.getpid() % 40, env=env, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "LLAMA_PIPELINE_OK" in proc.stdout
