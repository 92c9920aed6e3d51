"""The sharded optimizer composed with the other parallel dimensions, on gloo ranks (CPU):
hybrid sharding (``dp_replicate x dp_shard``), tensor parallel x sharded data parallel, a hybrid
optimizer whose "expert" part is sharded over a different group, and the global balancing
quantile. Every case is compared with plain single-process training on the same data."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from helpers import launch_ranks
import torch

ROOT = Path(__file__).resolve().parent.parent

PRELUDE = """
import torch, torch.distributed as dist
from torch.utils.data import DataLoader, TensorDataset
from ohara_b200.models.llama import Config, Llama
from ohara_b200.runtime import (EngineConfig, OharaEngine, ParallelConfig, StrategyType,
                                TensorParallelPlan)
from ohara_b200.optimizer import build_adamw, build_muon_adamw
from ohara_b200.trainer import Trainer
from ohara_b200.lr_scheduler import Scheduler

torch.manual_seed(0)
cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
             num_attention_heads=2, num_hidden_layers=2, dropout=0.0)
ids = torch.randint(0, 31, (8, 9))
dataset = TensorDataset(ids[:, :-1], ids[:, 1:])
base = Llama(cfg)
state = {k: v.clone() for k, v in base.state_dict().items()}

def reference(builder, steps=3):
    solo = Llama(cfg); solo.load_state_dict(state)
    opt = builder(solo)
    for _ in range(steps):
        loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
        loss.backward(); opt.step(); opt.zero_grad()
    return solo
"""


def _run(script, world, tmp_path, port_base=29300):
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(PRELUDE) + textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, world, port=port_base + os.getpid() % 500, env=env, timeout=400)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    return proc.stdout


def test_hybrid_sharding_replicate_times_shard_matches_single_process(tmp_path):
    """Four ranks as two replicas of a two-way sharded optimizer: shards over ``dp_shard``,
    reduced gradients averaged over ``dp_replicate``."""
    out = _run(
        """
        solo = reference(build_muon_adamw)
        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP,
                                          parallel=ParallelConfig(dp_replicate=2)))
        model = Llama(cfg); model.load_state_dict(state)
        model = engine.prepare(model)
        (opt,) = engine.prepare_optimizers(build_muon_adamw(model))
        assert opt.world == 2 and opt.replicate_world == 2, (opt.world, opt.replicate_world)
        assert engine.data_parallel_world_size == 4
        loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=2))
        trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                          max_iters=3, eval_iters=0, save_ckpt_iters=0, grad_clip_norm=1e9)
        trainer.train()
        for a, b in zip(solo.parameters(), model.parameters()):
            assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()
        if dist.get_rank() == 0:
            print("HSDP_OK")
        engine.close()
        """,
        4, tmp_path,
    )
    assert "HSDP_OK" in out


def test_tensor_parallel_times_sharded_optimizer_matches_single_process(tmp_path):
    """tp=2 x dp=2: every tensor-parallel rank shards its own slice of the model over its
    data-parallel peers; the clipped global norm counts tensor shards once each."""
    out = _run(
        """
        solo = Llama(cfg); solo.load_state_dict(state)
        ref_opt = build_adamw(solo, learning_rate=0.02, weight_decay=0.1)
        ref_norms = []
        for _ in range(3):
            loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
            loss.backward()
            ref_norms.append(float(torch.nn.utils.clip_grad_norm_(solo.parameters(), 0.5)))
            ref_opt.step(); ref_opt.zero_grad()
        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP,
                                          parallel=ParallelConfig(tp=2)))
        engine.launch()
        torch.manual_seed(100 + dist.get_rank())  # a different init on every rank:
        model = Llama(cfg)                        # the engine equalises it with rank 0's
        if dist.get_rank() == 0:
            model.load_state_dict(state)
        model = engine.prepare(model)
        assert engine.topology.tp == 2 and engine.topology.dp_shard == 2
        (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
        assert opt.world == 2
        loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=4))
        trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                          max_iters=3, eval_iters=0, save_ckpt_iters=0, grad_clip_norm=0.5)
        norms = []
        clip = engine.clip_gradients
        def recording(model, optimizer, max_norm):
            value = clip(model, optimizer, max_norm)
            norms.append(float(value))
            return value
        engine.clip_gradients = recording
        trainer.train()
        for got, want in zip(norms, ref_norms):
            assert abs(got - want) < 1e-4 * max(want, 1.0), (norms, ref_norms)
        full = engine.full_state_dict(model)
        for key, value in solo.state_dict().items():
            assert torch.allclose(full[key], value, atol=3e-5), (key, (full[key] - value).abs().max())
        if dist.get_rank() == 0:
            print("TP_FSDP_OK")
        engine.close()
        """,
        4, tmp_path, port_base=29900,
    )
    assert "TP_FSDP_OK" in out


def test_hybrid_optimizer_shards_each_part_over_its_own_group(tmp_path):
    """Two ranks; the feed-forward weights of layer 0 play the part of routed experts that only
    this rank holds (no replicas: ``solo``), everything else is sharded over both ranks. Dense
    gradients must be averaged over the ranks, "expert" gradients must stay local."""
    out = _run(
        """
        from ohara_b200.parallel.zero import HybridShardedOptimizer
        dist.init_process_group("gloo")
        rank = dist.get_rank()
        def tagged(model):
            for p in model.layers[0].ff.parameters():
                p.expert_parallel = True
            return model
        mine = ids[rank * 4:(rank + 1) * 4]
        # reference: plain optimizer fed the gradients the hybrid one should arrive at
        solo = tagged(Llama(cfg)); solo.load_state_dict(state)
        ref_opt = build_muon_adamw(solo)
        model = tagged(Llama(cfg)); model.load_state_dict(state)
        is_expert = lambda p: bool(getattr(p, "expert_parallel", False))
        opt = HybridShardedOptimizer(build_muon_adamw(model), [
            dict(select=lambda p: not is_expert(p)),
            dict(select=is_expert, solo=True, norm_groups={"ep": None}),
        ])
        assert [part.world for part in opt.parts] == [2, 1]
        for step in range(3):
            for m in (solo, model):
                (m.loss_sum(mine[:, :-1], mine[:, 1:]) / mine[:, 1:].numel()).backward()
            for p in solo.parameters():
                if not is_expert(p):
                    dist.all_reduce(p.grad); p.grad /= 2
            sq = sum(p.grad.square().sum() for p in solo.parameters() if not is_expert(p))
            local = sum(p.grad.square().sum() for p in solo.parameters() if is_expert(p))
            dist.all_reduce(local)                      # distinct "experts" on every rank
            want = float((sq + local).sqrt())
            got = float(opt.clip_grad_norm_(model, 1e9))
            assert abs(got - want) < 1e-4 * max(want, 1.0), (got, want)
            ref_opt.step(); ref_opt.zero_grad(); opt.step(); opt.zero_grad()
            for (name, a), b in zip(solo.named_parameters(), model.parameters()):
                assert torch.allclose(a, b, atol=2e-5), (step, name, (a - b).abs().max())
        blob = opt.state_dict()
        opt.load_state_dict(blob)
        if rank == 0:
            print("HYBRID_OK")
        dist.destroy_process_group()
        """,
        2, tmp_path, port_base=30500,
    )
    assert "HYBRID_OK" in out


def test_global_quantile_over_ranks_is_the_quantile_of_the_union(tmp_path):
    out = _run(
        """
        from ohara_b200.modules.routing import global_kth_largest
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        torch.manual_seed(7)
        everything = torch.randn(world, 300, 6) * torch.tensor([1.0, 5.0, 0.1]).view(3, 1, 1)
        everything[:, ::11] = 0.0
        for k in (1, 37, 450, 900):
            got = global_kth_largest(everything[rank], k)
            want = torch.topk(everything.reshape(-1, 6).t(), k, dim=-1).values[:, -1]
            assert torch.equal(got, want), (k, got, want)
        if rank == 0:
            print("QUANTILE_OK")
        dist.destroy_process_group()
        """,
        3, tmp_path, port_base=31100,
    )
    assert "QUANTILE_OK" in out


def test_pipeline_parallel_through_the_engine_matches_single_process(tmp_path):
    """pp=2 x dp=2 through ``OharaEngine`` and the ordinary ``Trainer``: every rank holds one
    stage, stages of one pipeline see the same batches, the sharded optimizer shards each stage
    over its data-parallel peers, the clipped norm spans both stages."""
    out = _run(
        """
        from ohara_b200.runtime import PipelinePlan
        solo = Llama(cfg); solo.load_state_dict(state)
        ref_opt = build_muon_adamw(solo)
        ref_norms, ref_losses = [], []
        for _ in range(3):
            loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
            loss.backward()
            ref_losses.append(float(loss))
            ref_norms.append(float(torch.nn.utils.clip_grad_norm_(solo.parameters(), 0.7)))
            ref_opt.step(); ref_opt.zero_grad()
        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP,
                                          parallel=ParallelConfig(pp=2),
                                          pipeline=PipelinePlan(degree=2, micro_batch_size=2)))
        model = Llama(cfg); model.load_state_dict(state)
        model = engine.prepare(model)
        assert type(model).__name__ == "PipelinedLlama"
        assert engine.data_parallel_world_size == 2
        (opt,) = engine.prepare_optimizers(build_muon_adamw(model))
        loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=4))
        trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                          max_iters=3, eval_iters=0, save_ckpt_iters=0, grad_clip_norm=0.7)
        norms, losses = [], []
        clip = engine.clip_gradients
        def recording(model, optimizer, max_norm):
            value = clip(model, optimizer, max_norm)
            norms.append(float(value))
            return value
        engine.clip_gradients = recording
        step = trainer.train_step
        def recording_step(idx):
            result = step(idx)
            losses.append(result[0])
            return result
        trainer.train_step = recording_step
        trainer.train()
        mean = torch.tensor(losses)          # a rank reports the loss of its own rows: the
        dist.all_reduce(mean); mean /= 4      # average over all ranks is the loss of the batch
        for got, want in zip(mean.tolist(), ref_losses):
            assert abs(got - want) < 1e-4 * max(abs(want), 1.0), (mean, ref_losses)
        for got, want in zip(norms, ref_norms):
            assert abs(got - want) < 1e-4 * max(want, 1.0), (norms, ref_norms)
        wanted = dict(solo.named_parameters())
        begin, end = model.stage.layer_range
        for name, p in model.stage.named_parameters():
            if name.startswith("layers."):
                index, rest = name.split(".", 2)[1:]
                name = f"layers.{int(index) + begin}.{rest}"
            assert torch.allclose(p, wanted[name], atol=3e-5), (name, (p - wanted[name]).abs().max())
        logits = model(ids[:2, :-1])
        assert torch.allclose(logits, solo(ids[:2, :-1]).float(), atol=1e-4)
        if dist.get_rank() == 0:
            print("PP_ENGINE_OK")
        engine.close()
        """,
        4, tmp_path, port_base=31700,
    )
    assert "PP_ENGINE_OK" in out


@pytest.mark.parametrize("builder,strategy,world", [
    ("build_muon_adamw", "FSDP", 4), ("build_muonh_adamh", "FSDP", 4),
    ("build_muonh_adamh", "DDP", 2),   # tp = world: the tensor-parallel group is the default group
])
def test_muon_on_tensor_parallel_shards_matches_the_unsharded_step(tmp_path, builder, strategy, world):
    """tp=2 x dp=2 with the Muon hybrid: the orthogonalisation runs on whole matrices gathered
    over the tensor-parallel group, every rank applies its slice; weights must follow the
    single-process run. The hyperspherical recipe (MuonH on hidden matrices, AdamH on the head)
    takes every norm over the whole matrix, so the shards stay on the whole matrix's sphere."""
    out = _run(
        f"""
        from ohara_b200.optimizer import build_muonh_adamh
        # the trainer's schedule is expressed in the builder's base rate (0.02 below)
        build = ({builder} if "{builder}" == "build_muon_adamw"
                 else (lambda m: build_muonh_adamh(m, learning_rate=0.02)))
        solo = reference(build)
        engine = OharaEngine(EngineConfig(strategy=StrategyType.{strategy},
                                          parallel=ParallelConfig(tp=2)))
        model = Llama(cfg); model.load_state_dict(state)
        model = engine.prepare(model)
        (opt,) = engine.prepare_optimizers(build(model))
        assert getattr(opt, "local", opt).tensor_parallel_world == 2
        loader = engine.prepare_dataloaders(
            DataLoader(dataset, batch_size=8 // engine.data_parallel_world_size))
        trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                          max_iters=3, eval_iters=0, save_ckpt_iters=0)
        trainer.train()
        full = engine.full_state_dict(model)
        for key, value in solo.state_dict().items():
            assert torch.allclose(full[key], value, atol=5e-5), (key, (full[key] - value).abs().max())
        if dist.get_rank() == 0:
            print("TP_MUON_OK")
        engine.close()
        """,
        world, tmp_path, port_base=32300,
    )
    assert "TP_MUON_OK" in out


def test_feed_forward_and_head_only_tensor_parallel_plan(tmp_path):
    """Four ranks on a model with two heads: the head count does not split, so only the
    feed-forward layers and the output head are sharded; logits must equal the unsharded model's
    on every rank."""
    out = _run(
        """
        engine = OharaEngine(EngineConfig(parallel=ParallelConfig(tp=4),
                                          tensor_parallel=TensorParallelPlan.mlp_and_head(4)))
        cfg32 = Config(vocab_size=32, max_sequence_length=8, hidden_size=16, intermediate_size=24,
                       num_attention_heads=2, num_hidden_layers=2, dropout=0.0)
        torch.manual_seed(3)
        whole = Llama(cfg32).eval()
        model = Llama(cfg32); model.load_state_dict(whole.state_dict())
        model = engine.prepare_module(model).eval()
        assert model.layers[0].ff.up.weight.shape == (24 // 4, 16)
        assert model.vocab_proj.weight.shape == (32 // 4, 16)
        assert model.layers[0].attn.query.weight.shape == (16, 16)       # attention replicated
        with torch.no_grad():
            got = model(ids[:, :-1])
            want = whole(ids[:, :-1])
        assert got.shape == want.shape
        assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()
        if dist.get_rank() == 0:
            print("MLP_HEAD_TP_OK")
        engine.close()
        """,
        4, tmp_path, port_base=32900,
    )
    assert "MLP_HEAD_TP_OK" in out


def test_tensor_parallel_ranks_without_data_parallel_peers_are_not_treated_as_replicas(tmp_path):
    """tp = world: there is no data-parallel group. Neither the sharded optimizer nor the DDP
    wrapper may fall back to the default group, which would average different tensor shards."""
    for strategy in ("FSDP", "DDP"):
        out = _run(
            f"""
            solo = reference(lambda m: build_adamw(m, learning_rate=0.02, weight_decay=0.1))
            engine = OharaEngine(EngineConfig(strategy=StrategyType.{strategy},
                                              parallel=ParallelConfig(tp=2),
                                              tensor_parallel=TensorParallelPlan.llama_default(2)))
            model = Llama(cfg); model.load_state_dict(state)
            model = engine.prepare(model)
            (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
            assert getattr(opt, "world", 1) == 1
            loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=8))
            trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                              max_iters=3, eval_iters=0, save_ckpt_iters=0)
            trainer.train()
            full = engine.full_state_dict(model)
            for name, value in solo.state_dict().items():
                assert torch.allclose(full[name], value, atol=2e-5), (name, (full[name] - value).abs().max())
            if dist.get_rank() == 0:
                print("TP_ONLY_OK")
            engine.close()
            """,
            2, tmp_path, port_base=29900,
        )
        assert "TP_ONLY_OK" in out


@pytest.mark.parametrize("shard_parameters", [False, True])
def test_checkpoint_of_a_tensor_parallel_run_resumes_in_a_fresh_engine_model(tmp_path, shard_parameters):
    """``engine.save`` writes whole tensors; ``engine.load`` cuts this rank's tensor-parallel slices
    back out, so a run resumed after two steps ends where four uninterrupted steps end."""
    out = _run(
        f"""
        import os, tempfile
        solo = reference(lambda m: build_adamw(m, learning_rate=0.02, weight_decay=0.1), steps=4)

        def make():
            model = Llama(cfg); model.load_state_dict(state)
            model = engine.prepare(model)
            (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
            loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=4))
            trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                              max_iters=2, eval_iters=0, save_ckpt_iters=0)
            return model, opt, trainer

        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP, parallel=ParallelConfig(tp=2),
                                          shard_parameters={shard_parameters},
                                          tensor_parallel=TensorParallelPlan.llama_default(2)))
        model, opt, trainer = make()
        trainer.train()
        folder = engine.broadcast(tempfile.mkdtemp() if dist.get_rank() == 0 else None)
        path = os.path.join(folder, "ckpt.pt")
        engine.save(path, trainer.checkpoint_state(2, 0.02, 0.0))
        model, opt, trainer = make()                      # fresh weights and optimizer state
        engine.load(path, {{"model": model, "optimizer": opt}})
        trainer.train()                                   # two more steps on the same batches
        full = engine.full_state_dict(model)
        for name, value in solo.state_dict().items():
            assert full[name].shape == value.shape, name
            assert torch.allclose(full[name], value, atol=3e-5), (name, (full[name] - value).abs().max())
        if dist.get_rank() == 0:
            print("TP_RESUME_OK")
        engine.close()
        """,
        4, tmp_path, port_base=30100,
    )
    assert "TP_RESUME_OK" in out


def test_checkpoint_of_a_pipeline_run_is_a_whole_model_and_resumes(tmp_path):
    """pp=2 x dp=2: the saved model state has the whole model's keys (it loads into a plain
    Llama), the optimizer state is kept per stage, and a fresh engine model resumes from it."""
    out = _run(
        """
        import os, tempfile
        from ohara_b200.runtime import PipelinePlan
        solo = reference(lambda m: build_adamw(m, learning_rate=0.02, weight_decay=0.1), steps=4)
        half = reference(lambda m: build_adamw(m, learning_rate=0.02, weight_decay=0.1), steps=2)

        def make():
            model = Llama(cfg); model.load_state_dict(state)
            model = engine.prepare(model)
            (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
            loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=4))
            trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                              max_iters=2, eval_iters=0, save_ckpt_iters=0)
            return model, opt, trainer

        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP, parallel=ParallelConfig(pp=2),
                                          pipeline=PipelinePlan(degree=2, micro_batch_size=2)))
        model, opt, trainer = make()
        trainer.train()
        full = engine.full_state_dict(model)
        assert set(full) == set(half.state_dict()), set(full) ^ set(half.state_dict())
        plain = Llama(cfg); plain.load_state_dict(full)              # loads into the plain model
        for name, value in half.state_dict().items():
            assert torch.allclose(full[name], value, atol=3e-5), name
        folder = engine.broadcast(tempfile.mkdtemp() if dist.get_rank() == 0 else None)
        path = os.path.join(folder, "ckpt.pt")
        engine.save(path, trainer.checkpoint_state(2, 0.02, 0.0))
        model, opt, trainer = make()
        engine.load(path, {"model": model, "optimizer": opt})
        trainer.train()
        full = engine.full_state_dict(model)
        for name, value in solo.state_dict().items():
            assert torch.allclose(full[name], value, atol=3e-5), (name, (full[name] - value).abs().max())
        if dist.get_rank() == 0:
            print("PP_RESUME_OK")
        engine.close()
        """,
        4, tmp_path, port_base=30300,
    )
    assert "PP_RESUME_OK" in out


@pytest.mark.parametrize("world,ep", [(4, 2)])
def test_expert_parallel_training_on_cpu_ranks_matches_single_process_and_resumes(tmp_path, world, ep):
    """ep=2 (x dp=2): every rank keeps half of the routed experts and exchanges rows with
    all-to-alls (the process-group form of the expert-parallel layer); dense parameters are sharded
    over all ranks, experts over the ranks that hold the same ones; the checkpoint holds all
    experts and one optimizer state per expert-parallel coordinate."""
    out = _run(
        f"""
        import os, tempfile
        moe_cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
                         num_attention_heads=2, num_hidden_layers=2, dropout=0.0, moe_num_experts=4,
                         moe_experts_per_tok=2, moe_grouped=True, moe_num_shared_experts=1)
        moe_state = {{k: v.clone() for k, v in Llama(moe_cfg).state_dict().items()}}
        for name in moe_state:                         # the routed output projections start at zero
            if name.endswith("w_down"):
                moe_state[name].normal_(std=0.1)

        def solo_after(steps):
            solo = Llama(moe_cfg); solo.load_state_dict(moe_state)
            opt = build_adamw(solo, learning_rate=0.02, weight_decay=0.1)
            for _ in range(steps):
                loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
                loss.backward(); opt.step(); opt.zero_grad()
            return solo

        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP, parallel=ParallelConfig(ep={ep})))

        def make():
            model = Llama(moe_cfg); model.load_state_dict(moe_state)
            model = engine.prepare(model)
            (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
            replicas = engine.data_parallel_world_size
            loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=8 // replicas))
            trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                              max_iters=2, eval_iters=0, save_ckpt_iters=0)
            return model, opt, trainer

        def close_to(model, solo):
            full = engine.full_state_dict(model)
            for name, value in solo.state_dict().items():
                assert full[name].shape == value.shape, (name, full[name].shape, value.shape)
                assert torch.allclose(full[name], value, atol=3e-5), (name, (full[name] - value).abs().max())

        model, opt, trainer = make()
        assert engine.data_parallel_world_size == {world}
        assert model.layers[0].ff.w_gate.shape[0] == 4 // {ep}
        assert type(opt).__name__ == "HybridShardedOptimizer"
        trainer.train()
        close_to(model, solo_after(2))
        folder = engine.broadcast(tempfile.mkdtemp() if dist.get_rank() == 0 else None)
        path = os.path.join(folder, "ckpt.pt")
        engine.save(path, trainer.checkpoint_state(2, 0.02, 0.0))
        model, opt, trainer = make()
        engine.load(path, {{"model": model, "optimizer": opt}})
        trainer.train()
        close_to(model, solo_after(4))
        if dist.get_rank() == 0:
            print("EP_CPU_OK")
        engine.close()
        """,
        world, tmp_path, port_base=30500,
    )
    assert "EP_CPU_OK" in out


@pytest.mark.parametrize("strategy,shard_parameters,world", [
    ("DDP", False, 2), ("FSDP", True, 2)])
def test_sequence_parallel_layout_over_the_process_group(tmp_path, strategy, shard_parameters, world):
    """``sequence_parallel=True`` without peer memory: every tensor-parallel rank works on its
    B / tp sequences between the parallel regions (the engine slices the batch and scales the
    loss), column-parallel layers all-gather the token blocks, row-parallel layers reduce-scatter
    them, and replicated parameters (norms, embedding) sum their partial gradients over the
    group: under DDP, under the sharded optimizer and under sharded parameters (tp = world in the
    two-rank cases, where the tensor-parallel group is the default group)."""
    out = _run(
        f"""
        solo = Llama(cfg); solo.load_state_dict(state)
        ref_opt = build_adamw(solo, learning_rate=0.02, weight_decay=0.1)
        ref_norms = []
        for _ in range(3):
            loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
            loss.backward()
            ref_norms.append(float(torch.nn.utils.clip_grad_norm_(solo.parameters(), 0.5)))
            ref_opt.step(); ref_opt.zero_grad()
        engine = OharaEngine(EngineConfig(
            strategy=StrategyType.{strategy}, shard_parameters={shard_parameters},
            parallel=ParallelConfig(tp=2),
            tensor_parallel=TensorParallelPlan.llama_default(2, sequence_parallel=True)))
        model = Llama(cfg); model.load_state_dict(state)
        model = engine.prepare(model)
        (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
        batch = 8 // engine.data_parallel_world_size
        local = engine.local_batch((ids[:batch, :-1], ids[:batch, 1:]))
        assert local[0].shape[0] == batch // 2                      # this rank's sequences
        loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=batch))
        trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                          max_iters=3, eval_iters=0, save_ckpt_iters=0, grad_clip_norm=0.5)
        norms = []
        clip = engine.clip_gradients
        def recording(m, o, max_norm):
            value = clip(m, o, max_norm); norms.append(float(value)); return value
        engine.clip_gradients = recording
        trainer.train()
        assert all(abs(a - b) < 1e-4 * max(1.0, b) for a, b in zip(norms, ref_norms)), (norms, ref_norms)
        full = engine.full_state_dict(model)
        for name, value in solo.state_dict().items():
            assert torch.allclose(full[name], value, atol=3e-5), (name, (full[name] - value).abs().max())
        if dist.get_rank() == 0:
            print("SP_C10D_OK")
        engine.close()
        """,
        world, tmp_path, port_base=30700,
    )
    assert "SP_C10D_OK" in out
