"""Runtime: topology arithmetic, tensor-parallel plan, engine facade, multi-process (gloo) paths."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from helpers import launch_ranks
import torch

from ohara_b200.runtime import (
    EngineConfig,
    OharaEngine,
    ParallelConfig,
    ParallelTopology,
    PipelinePlan,
    PipelineStageSpec,
    ReduceType,
    TensorParallelPlan,
    TensorParallelStyle,
)

ROOT = Path(__file__).resolve().parent.parent


def test_topology_infers_dp_shard_and_validates():
    topo = ParallelTopology.from_config(8, ParallelConfig(tp=2))
    assert topo.dp_shard == 4 and topo.dp_world_size == 4
    with pytest.raises(ValueError):
        ParallelTopology.from_config(6, ParallelConfig(tp=4))
    with pytest.raises(ValueError):
        ParallelTopology(world_size=8, dp_replicate=1, dp_shard=3, tp=2, pp=1, cp=1, ep=1)
    with pytest.raises(ValueError):
        ParallelTopology(world_size=0, dp_replicate=1, dp_shard=0, tp=1, pp=1, cp=1, ep=1)


def test_rank_order_is_pp_dp_cp_tp_ep():
    topo = ParallelTopology(world_size=16, dp_replicate=1, dp_shard=2, tp=2, pp=2, cp=2, ep=1)
    assert topo.tensor_parallel_group_ranks(0) == [0, 1]
    assert topo.context_parallel_group_ranks(0) == [0, 2]
    assert topo.data_parallel_group_ranks(0) == [0, 4]
    assert topo.group_ranks("pp", 0) == [0, 8]
    assert topo.tensor_parallel_group_ranks(13) == [12, 13]
    groups = list(topo.iter_all_data_parallel_groups())
    assert sorted(r for g in groups for r in g) == list(range(16)) and len(groups) == 8
    for rank in range(16):
        assert topo._rank_from_coordinates(topo._coordinates(rank)) == rank


def test_tp_ranks_share_a_data_rank(monkeypatch):
    topo = ParallelTopology.from_config(8, ParallelConfig(tp=4))
    seen = {}
    for rank in range(8):
        monkeypatch.setenv("RANK", str(rank))
        seen[rank] = (topo.dp_rank, topo.tp_rank)
    assert [seen[r][0] for r in range(8)] == [0, 0, 0, 0, 1, 1, 1, 1]
    assert [seen[r][1] for r in range(8)] == [0, 1, 2, 3, 0, 1, 2, 3]
    monkeypatch.setenv("RANK", "7")
    assert not topo.is_first_pp_stage or topo.pp == 1


def test_tensor_parallel_plan_rules():
    plan = TensorParallelPlan.llama_default(4)
    assert plan.style_for("layers.3.attn.query") == TensorParallelStyle.COLWISE
    assert plan.style_for("layers.11.ff.down") == TensorParallelStyle.ROWWISE
    assert plan.style_for("vocab_proj") is None
    plan.validate(hidden_size=768)
    with pytest.raises(ValueError):
        plan.validate(hidden_size=770)
    with pytest.raises(ValueError):
        TensorParallelPlan(degree=0).validate()


def test_pipeline_plan_validation():
    plan = PipelinePlan(degree=2, micro_batch_size=2, stages=[PipelineStageSpec(["a"]) for _ in range(4)])
    plan.validate(local_batch_size=8)
    assert len(plan.stages_for_rank(1)) == 2
    with pytest.raises(ValueError):
        plan.validate(local_batch_size=7)
    with pytest.raises(ValueError):
        PipelinePlan(degree=2, stages=[PipelineStageSpec(["a"])] * 3).validate(2)
    with pytest.raises(ValueError):
        PipelinePlan(degree=0).validate(1)


def test_engine_single_process_facade(tmp_path):
    engine = OharaEngine()
    assert engine.launch(lambda a, b=1: a + b, 2, b=3) == 5
    assert engine.launched and engine.world_size == 1 and engine.is_global_zero
    batch = {"x": torch.ones(2), "y": [torch.zeros(1), (torch.ones(1), 3)]}
    moved = engine.to_device(batch)
    assert moved["y"][1][1] == 3 and moved["x"].device == engine.device
    t = torch.tensor([2.0])
    assert engine.all_reduce(t, ReduceType.MEAN) is t
    assert engine.all_gather(t)[0] is t
    assert engine.broadcast({"a": 1}) == {"a": 1}
    with pytest.raises(ValueError):
        engine.all_reduce(t, "product")
    with pytest.raises(ValueError):
        engine.prepare_dataloaders()
    logged = []

    class Sink:
        def log_metrics(self, payload, step=None):
            logged.append((payload, step))

    engine.loggers.append(Sink())
    engine.log_dict({"loss": 1.0}, step=3)
    assert logged == [({"loss": 1.0}, 3)]
    model = torch.nn.Linear(2, 2)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    same_model, same_opt = engine.setup(model, opt)
    assert same_model is model and same_opt is opt
    engine.save(tmp_path / "a" / "b.pt", {"k": 1})
    assert engine.load(tmp_path / "a" / "b.pt")["k"] == 1


def _run_ranks(script: str, world: int, tmp_path, timeout=240):
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, world, port=29500 + os.getpid() % 500, env=env, timeout=timeout)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    return proc.stdout


def test_tensor_parallel_matches_single_device_on_two_ranks(tmp_path):
    out = _run_ranks(
        """
        import torch, torch.distributed as dist
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, ParallelConfig
        torch.manual_seed(0)
        cfg = Config(vocab_size=50, max_sequence_length=16, hidden_size=32, intermediate_size=48,
                     num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, dropout=0.0)
        reference = Llama(cfg)
        ids = torch.randint(0, 50, (2, 12))
        ref_loss = reference.loss_sum(ids[:, :-1], ids[:, 1:])
        ref_loss.backward()
        engine = OharaEngine(EngineConfig(parallel=ParallelConfig(tp=2)))
        model = Llama(cfg)
        model.load_state_dict(reference.state_dict())
        model = engine.prepare(model)
        assert engine.topology.tp == 2 and engine.data_parallel_world_size == 1
        loss = model.loss_sum(ids[:, :-1], ids[:, 1:])
        loss.backward()
        assert torch.allclose(loss, ref_loss, rtol=1e-4), (loss, ref_loss)
        rank = dist.get_rank()
        q_ref = reference.layers[0].attn.query.weight.grad.chunk(2, 0)[rank]
        assert torch.allclose(model.layers[0].attn.query.weight.grad, q_ref, atol=1e-4)
        d_ref = reference.layers[1].ff.down.weight.grad.chunk(2, 1)[rank]
        assert torch.allclose(model.layers[1].ff.down.weight.grad, d_ref, atol=1e-4)
        assert torch.allclose(model.norm.weight.grad, reference.norm.weight.grad, atol=1e-4)
        full = engine.full_state_dict(model)
        for key, value in reference.state_dict().items():
            assert torch.equal(full[key], value), key
        if rank == 0:
            print("TP_OK")
        engine.close()
        """,
        2, tmp_path,
    )
    assert "TP_OK" in out


def test_ddp_two_ranks_match_single_process(tmp_path):
    out = _run_ranks(
        """
        import torch, torch.distributed as dist
        from torch.utils.data import DataLoader, TensorDataset
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import OharaEngine
        from ohara_b200.optimizer import build_adamw
        from ohara_b200.trainer import Trainer
        from ohara_b200.lr_scheduler import Scheduler
        torch.manual_seed(0)
        cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
                     num_attention_heads=2, num_hidden_layers=1, dropout=0.0)
        ids = torch.randint(0, 31, (8, 9))
        ds = TensorDataset(ids[:, :-1], ids[:, 1:])
        base = Llama(cfg)
        state = {k: v.clone() for k, v in base.state_dict().items()}
        # single process, full batch
        solo = Llama(cfg); solo.load_state_dict(state)
        opt = build_adamw(solo, learning_rate=1e-2, weight_decay=0.0)
        loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
        loss.backward(); opt.step()
        engine = OharaEngine()
        model = Llama(cfg); model.load_state_dict(state)
        model = engine.prepare(model)
        assert engine.data_parallel_world_size == 2
        opt2 = build_adamw(model, learning_rate=1e-2, weight_decay=0.0)
        dl = engine.prepare_dataloaders(DataLoader(ds, batch_size=4))
        trainer = Trainer(engine, model, opt2, dl, dl, Scheduler(1e-2), micro_batch=1, max_iters=1,
                          eval_iters=0, save_ckpt_iters=0)
        trainer.train()
        for a, b in zip(solo.parameters(), model.module.parameters()):
            assert torch.allclose(a, b, atol=1e-5)
        if dist.get_rank() == 0:
            print("DDP_OK")
        engine.close()
        """,
        2, tmp_path,
    )
    assert "DDP_OK" in out
