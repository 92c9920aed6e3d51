"""Parameter sharding per transformer block: gathered just in time, released after use, gradients
reduce-scattered per unit. Single-process cases check the bookkeeping; gloo ranks check that
training matches a single process on the same data."""

import copy
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from helpers import launch_ranks
import torch

from ohara_b200 import Config, Llama
from ohara_b200.optimizer import build_adamw, build_muon_adamw
from ohara_b200.parallel.param_shard import ParameterShardedOptimizer, shard_llama

ROOT = Path(__file__).resolve().parent.parent


def _config(**extra) -> Config:
    return Config(vocab_size=37, max_sequence_length=16, hidden_size=32, intermediate_size=40,
                  num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3, dropout=0.0,
                  **extra)


def _train(model, optimizer, tokens, steps, micro=1, finish=None):
    losses = []
    for _ in range(steps):
        for part in tokens.chunk(micro):
            loss = model(part[:, :-1], targets=part[:, 1:]) / tokens[:, 1:].numel()
            loss.backward()
            if finish is not None:
                finish()
            losses.append(float(loss.detach()))
        optimizer.step()
        optimizer.zero_grad()
    return losses


@pytest.mark.parametrize("variant", ["dense", "tied", "moe", "checkpointed", "micro"])
def test_sharded_model_trains_like_the_plain_model(variant):
    extra = {}
    if variant == "tied":
        extra["weight_tying"] = True
    if variant == "moe":
        extra.update(moe_num_experts=4, moe_experts_per_tok=2, moe_grouped=True,
                     moe_num_shared_experts=1, moe_aux_loss_coef=0.01)
    torch.manual_seed(0)
    plain = Llama(_config(**extra))
    sharded = copy.deepcopy(plain)
    if variant == "checkpointed":
        sharded.enable_activation_checkpointing()
    tokens = torch.randint(0, 37, (4, 13))
    micro = 2 if variant == "micro" else 1
    plain_opt = build_adamw(plain, learning_rate=1e-2, weight_decay=0.1)
    sharding = shard_llama(sharded)
    sharded_opt = ParameterShardedOptimizer(
        build_adamw(sharded, learning_rate=1e-2, weight_decay=0.1), sharding)
    plain.train(), sharded.train()
    want = _train(plain, plain_opt, tokens, 3, micro)
    got = _train(sharded, sharded_opt, tokens, 3, micro, finish=sharding.finish_backward)
    assert got == pytest.approx(want, rel=1e-5, abs=1e-6)
    state = sharding.full_state_dict(sharded)
    for name, value in plain.state_dict().items():
        torch.testing.assert_close(state[name], value, rtol=1e-5, atol=1e-6, msg=name)


def test_parameters_are_placeholders_between_uses_and_keep_their_shape():
    torch.manual_seed(0)
    model = Llama(_config())
    shapes = {n: tuple(p.shape) for n, p in model.named_parameters()}
    count = sum(p.numel() for p in model.parameters())
    sharding = shard_llama(model)
    for name, p in model.named_parameters():
        assert tuple(p.shape) == shapes[name] and p.ndim == len(shapes[name])
        assert p.untyped_storage().nbytes() == 4, name            # one element, expanded
    assert sum(p.numel() for p in model.parameters()) == count
    # decay / no-decay partition by dimensionality still works on the placeholders
    optimizer = build_adamw(model, learning_rate=1e-3, weight_decay=0.1)
    assert sum(len(g["params"]) for g in optimizer.param_groups) == len(shapes)
    tokens = torch.randint(0, 37, (2, 9))
    model.train()
    loss = model(tokens[:, :-1], targets=tokens[:, 1:])
    gathered_after_forward = [u.name for u in sharding.units if u.full is not None]
    assert gathered_after_forward == ["layers.2", "head"]       # the last block and the head stay
    loss.backward()
    sharding.finish_backward()
    assert all(u.full is None for u in sharding.units)
    assert all(p.grad is None for p in model.parameters())        # full gradients are dropped
    assert all(u.grad is not None and u.grad.numel() == u.region for u in sharding.units)
    report = sharding.memory_report()
    assert report["unsharded_bytes"] == count * 4
    largest_two = sum(sorted(u.total for u in sharding.units)[-2:]) * 4
    assert report["peak_gathered_bytes"] <= largest_two + max(u.total for u in sharding.units) * 4


def test_evaluation_pass_releases_the_blocks():
    torch.manual_seed(0)
    model = Llama(_config())
    reference = copy.deepcopy(model).eval()
    sharding = shard_llama(model)
    model.eval()
    tokens = torch.randint(0, 37, (2, 9))
    with torch.no_grad():
        torch.testing.assert_close(model(tokens), reference(tokens))
        assert all(u.full is None for u in sharding.units)      # the head too, once it was used
        want = reference.loss_sum(tokens[:, :-1], tokens[:, 1:])
        torch.testing.assert_close(model.loss_sum(tokens[:, :-1], tokens[:, 1:]), want)
    assert all(u.full is None for u in sharding.units)
    with pytest.raises(NotImplementedError, match="whole parameters"):
        model(tokens[:, :1], model.build_kv_cache(batch_size=2), 0)


def test_loop_moe_units_are_deferred_and_muon_runs_on_one_process_with_either_layout():
    torch.manual_seed(0)
    loop = Llama(_config(moe_num_experts=4, moe_experts_per_tok=2))
    assert all(u.deferred == u.name.startswith("layers.") for u in shard_llama(loop).units)
    with pytest.raises(ValueError):
        shard_llama(Llama(_config()), layout="diagonal")
    # one process owns everything, so whole-matrix groups are fine whatever the layout
    tokens = torch.randint(0, 37, (4, 13))
    base = Llama(_config())
    plain = copy.deepcopy(base)
    want = _train(plain.train(), build_muon_adamw(plain), tokens, 3)
    for layout in ("even", "matrix"):
        model = copy.deepcopy(base)
        sharding = shard_llama(model, layout=layout)
        optimizer = ParameterShardedOptimizer(build_muon_adamw(model), sharding)
        got = _train(model.train(), optimizer, tokens, 3, finish=sharding.finish_backward)
        assert got == pytest.approx(want, rel=1e-5, abs=1e-6)


def test_matrix_layout_keeps_every_block_parameter_inside_one_region():
    from ohara_b200.parallel.param_shard import _Unit

    torch.manual_seed(0)
    block = Llama(_config()).layers[0]
    params = list(block.parameters())
    for world in (2, 3, 8):
        units = [_Unit("layers.0", params, world, rank, True, whole_tensors=True)
                 for rank in range(world)]
        unit = units[0]
        assert unit.total == unit.region * world
        spans = sorted((off, off + n) for off, n in zip(unit.offsets, unit.numels))
        assert all(a_end <= b_begin for (_, a_end), (b_begin, _) in zip(spans, spans[1:]))  # disjoint
        for off, n in zip(unit.offsets, unit.numels):
            assert off // unit.region == (off + n - 1) // unit.region                   # one owner
        # the masters of the ranks tile the flat vector
        flat = torch.cat([u.master for u in units])
        for p, off, n in zip(params, unit.offsets, unit.numels):
            assert torch.equal(flat[off:off + n], p.detach().reshape(-1))
        even = _Unit("layers.0", params, world, 0, True)
        assert unit.total >= even.total
        owners = {off // unit.region for off in unit.offsets}
        assert len(owners) == min(world, len(params)) or world > len(params)


def test_state_dict_round_trip_and_clipping():
    torch.manual_seed(0)
    model = Llama(_config())
    plain = copy.deepcopy(model)
    sharding = shard_llama(model)
    optimizer = ParameterShardedOptimizer(build_adamw(model, learning_rate=1e-2, weight_decay=0.0), sharding)
    plain_opt = build_adamw(plain, learning_rate=1e-2, weight_decay=0.0)
    tokens = torch.randint(0, 37, (2, 9))
    model.train(), plain.train()
    for m in (model, plain):
        m(tokens[:, :-1], targets=tokens[:, 1:]).backward()
    norm = optimizer.clip_grad_norm_(model, 0.5)
    want = torch.nn.utils.clip_grad_norm_(plain.parameters(), 0.5)
    torch.testing.assert_close(norm, want, rtol=1e-5, atol=1e-6)
    optimizer.step(), plain_opt.step()
    saved = copy.deepcopy(optimizer.state_dict())
    full = sharding.full_state_dict(model)
    for name, value in plain.state_dict().items():
        torch.testing.assert_close(full[name], value, rtol=1e-5, atol=1e-6, msg=name)
    # a fresh sharded model restored from the full weights and the optimizer shard continues alike
    again = Llama(_config())
    again_sharding = shard_llama(again)
    again_sharding.load_full_state_dict(again, full)
    again_opt = ParameterShardedOptimizer(build_adamw(again, learning_rate=1e-2, weight_decay=0.0), again_sharding)
    again_opt.load_state_dict(saved)
    again.train()
    for m, o in ((model, optimizer), (again, again_opt)):
        o.zero_grad()
        m(tokens[:, :-1], targets=tokens[:, 1:]).backward()
        o.step()
    a, b = sharding.full_state_dict(model), again_sharding.full_state_dict(again)
    for name in a:
        torch.testing.assert_close(a[name], b[name], rtol=1e-6, atol=1e-7, msg=name)


WORKER = """
import torch, torch.distributed as dist
from torch.utils.data import DataLoader, TensorDataset
from ohara_b200.models.llama import Config, Llama
from ohara_b200.runtime import EngineConfig, OharaEngine, StrategyType
from ohara_b200.optimizer import build_adamw
from ohara_b200.trainer import Trainer
from ohara_b200.lr_scheduler import Scheduler

torch.manual_seed(0)
cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
             num_attention_heads=2, num_hidden_layers=3, dropout=0.0)
ids = torch.randint(0, 31, (8, 9))
dataset = TensorDataset(ids[:, :-1], ids[:, 1:])
state = {k: v.clone() for k, v in Llama(cfg).state_dict().items()}

solo = Llama(cfg); solo.load_state_dict(state)
ref_opt = build_adamw(solo, learning_rate=0.02, weight_decay=0.1)
ref_norms = []
for _ in range(4):
    loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
    loss.backward()
    ref_norms.append(float(torch.nn.utils.clip_grad_norm_(solo.parameters(), 0.5)))
    ref_opt.step(); ref_opt.zero_grad()

engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP, shard_parameters=True,
                                  activation_checkpointing=CHECKPOINT))
model = Llama(cfg); model.load_state_dict(state)
model = engine.prepare(model)
(opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
assert type(opt).__name__ == "ParameterShardedOptimizer"
world = dist.get_world_size()
report = model._param_sharding.memory_report()
assert report["persistent_bytes_per_rank"] * world < report["unsharded_bytes"] * 1.25 + 4096 * world
loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=8 // world // MICRO))
trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=MICRO,
                  max_iters=4, eval_iters=0, save_ckpt_iters=0, grad_clip_norm=0.5)
norms = []
clip = opt.clip_grad_norm_
opt.clip_grad_norm_ = lambda m, n: (norms.append(float(clip(m, n))), norms[-1])[1] and torch.tensor(norms[-1])
trainer.train()
assert all(abs(a - b) < 1e-4 * max(1.0, abs(b)) for a, b in zip(norms, ref_norms)), (norms, ref_norms)
full = engine.full_state_dict(model)
for name, value in solo.state_dict().items():
    assert torch.allclose(full[name], value, atol=3e-5), (name, (full[name] - value).abs().max())
assert all(u.full is None for u in model._param_sharding.units)

# checkpoint written by rank 0, restored into a fresh sharded model + optimizer on every rank
import os, tempfile
folder = engine.broadcast(tempfile.mkdtemp() if dist.get_rank() == 0 else None)
path = os.path.join(folder, "ckpt.pt")
engine.save(path, trainer.checkpoint_state(4, 0.02, 0.0))
fresh = engine.prepare(Llama(cfg))
(fresh_opt,) = engine.prepare_optimizers(build_adamw(fresh, learning_rate=0.02, weight_decay=0.1))
engine.load(path, {"model": fresh, "optimizer": fresh_opt})
restored = engine.full_state_dict(fresh)
for name, value in full.items():
    assert torch.equal(restored[name], value), name
a, b = opt.local.state_dict()["state"], fresh_opt.local.state_dict()["state"]
assert a.keys() == b.keys() and len(a) > 0
for key in a:
    assert torch.equal(a[key]["exp_avg"], b[key]["exp_avg"])
if dist.get_rank() == 0:
    print("PARAM_SHARD_OK", report)
engine.close()
"""


@pytest.mark.parametrize("world,micro,checkpoint", [(4, 2, False)])
def test_gloo_ranks_match_single_process_training(tmp_path, world, micro, checkpoint):
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(WORKER).replace("MICRO", str(micro))
                    .replace("CHECKPOINT", str(checkpoint)))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, world, port=29800 + os.getpid() % 150, env=env, timeout=400)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "PARAM_SHARD_OK" in proc.stdout


RESHARD_WORKER = """
import sys, torch, torch.distributed as dist
from ohara_b200.models.llama import Config, Llama
from ohara_b200.runtime import EngineConfig, OharaEngine, StrategyType
from ohara_b200.optimizer import build_adamw

torch.manual_seed(0)
cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
             num_attention_heads=2, num_hidden_layers=3, dropout=0.0)
ids = torch.randint(0, 31, (8, 9))
engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP, shard_parameters=True))
model = engine.prepare(Llama(cfg))
(opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
rank, world = dist.get_rank(), dist.get_world_size()
rows = ids[rank * (8 // world):(rank + 1) * (8 // world)]
model.train()
for _ in range(2):
    loss = model(rows[:, :-1], targets=rows[:, 1:]) / rows[:, 1:].numel()
    engine.backward(loss); opt.step(); opt.zero_grad()
engine.save(sys.argv[1], {"model": engine.full_state_dict(model), "optimizer": opt.state_dict(),
                          "ids": ids})
engine.close()
"""


def test_checkpoint_of_two_ranks_continues_in_one_process(tmp_path):
    """The optimizer state is stored per unit as whole vectors, so a run saved on two ranks
    resumes on one (and the resumed run equals four uninterrupted single-process steps)."""
    path, checkpoint = tmp_path / "worker.py", tmp_path / "ckpt.pt"
    path.write_text(textwrap.dedent(RESHARD_WORKER))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, 2, port=31200 + os.getpid() % 150, env=env, timeout=400,
                        args=(str(checkpoint),))
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    saved = torch.load(checkpoint, weights_only=False)
    ids = saved["ids"]
    cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
                 num_attention_heads=2, num_hidden_layers=3, dropout=0.0)
    torch.manual_seed(0)                      # the worker's random stream: tokens, then weights
    assert torch.equal(torch.randint(0, 31, (8, 9)), ids)
    plain = Llama(cfg)
    plain_opt = build_adamw(plain, learning_rate=0.02, weight_decay=0.1)
    plain.train()
    for _ in range(4):
        (plain(ids[:, :-1], targets=ids[:, 1:]) / ids[:, 1:].numel()).backward()
        plain_opt.step()
        plain_opt.zero_grad()
    resumed = Llama(cfg)
    sharding = shard_llama(resumed)
    sharding.load_full_state_dict(resumed, saved["model"])
    optimizer = ParameterShardedOptimizer(
        build_adamw(resumed, learning_rate=0.02, weight_decay=0.1), sharding)
    optimizer.load_state_dict(saved["optimizer"])
    resumed.train()
    for _ in range(2):
        (resumed(ids[:, :-1], targets=ids[:, 1:]) / ids[:, 1:].numel()).backward()
        optimizer.step()
        optimizer.zero_grad()
    final = sharding.full_state_dict(resumed)
    for name, value in plain.state_dict().items():
        torch.testing.assert_close(final[name], value, rtol=1e-4, atol=3e-5, msg=name)


COMPOSED_WORKER = """
import torch, torch.distributed as dist
from torch.utils.data import DataLoader, TensorDataset
from ohara_b200.models.llama import Config, Llama
from ohara_b200.runtime import (EngineConfig, OharaEngine, ParallelConfig, StrategyType,
                                TensorParallelPlan)
from ohara_b200.optimizer import build_adamw
from ohara_b200.trainer import Trainer
from ohara_b200.lr_scheduler import Scheduler

torch.manual_seed(0)
cfg = Config(vocab_size=32, max_sequence_length=16, hidden_size=16, intermediate_size=24,
             num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, dropout=0.0)
ids = torch.randint(0, 32, (8, 17))
dataset = TensorDataset(ids[:, :-1], ids[:, 1:])
state = {k: v.clone() for k, v in Llama(cfg).state_dict().items()}
solo = Llama(cfg); solo.load_state_dict(state)
ref_opt = build_adamw(solo, learning_rate=0.02, weight_decay=0.1)
ref_norms = []
for _ in range(3):
    loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
    loss.backward()
    ref_norms.append(float(torch.nn.utils.clip_grad_norm_(solo.parameters(), 0.5)))
    ref_opt.step(); ref_opt.zero_grad()

engine = OharaEngine(EngineConfig(
    strategy=StrategyType.FSDP, shard_parameters=SHARD, context_parallel_mode="ulysses",
    activation_checkpointing=RECOMPUTE, parallel=ParallelConfig(tp=TP, cp=CP, dp_replicate=REPLICAS),
    tensor_parallel=TensorParallelPlan.llama_default(TP) if TP > 1 else TensorParallelPlan()))
model = Llama(cfg); model.load_state_dict(state)
model = engine.prepare(model)
(opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.1))
assert (type(opt).__name__ == "ParameterShardedOptimizer") == SHARD
dp = engine.data_parallel_world_size
assert dp == dist.get_world_size() // (TP * CP)
loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=8 // dp))
trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                  max_iters=3, eval_iters=0, save_ckpt_iters=0, grad_clip_norm=0.5)
norms = []
clip = opt.clip_grad_norm_
def recording(m, n):
    value = clip(m, n); norms.append(float(value)); return value
opt.clip_grad_norm_ = recording
trainer.train()
assert all(abs(a - b) < 1e-4 * max(1.0, abs(b)) for a, b in zip(norms, ref_norms)), (norms, ref_norms)
full = engine.full_state_dict(model)
for name, value in solo.state_dict().items():
    assert full[name].shape == value.shape, name
    assert torch.allclose(full[name], value, atol=3e-5), (name, (full[name] - value).abs().max())
if dist.get_rank() == 0:
    print("COMPOSED_OK")
engine.close()
"""


@pytest.mark.parametrize("world,tp,cp,shard,recompute,replicas", [
    (4, 1, 2, True, False, 1), (2, 2, 1, True, False, 1),
    (4, 1, 1, True, False, 2),  # hybrid sharding: two replicas of a two-way sharded model
    (4, 2, 1, True, True, 1),   # sharded parameters + recomputed blocks under tensor parallelism
])
def test_sharded_parameters_compose_with_tensor_and_context_parallelism(tmp_path, world, tp, cp,
                                                                        shard, recompute, replicas):
    """The units are this rank's tensor shards, sharded over its data- and context-parallel
    peers; the clipped global norm counts tensor shards once each. Recomputed blocks repeat their
    collectives in the backward pass, on every rank at the same point."""
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(COMPOSED_WORKER).replace("TP", str(tp)).replace("CP", str(cp))
                    .replace("SHARD", str(shard)).replace("RECOMPUTE", str(recompute))
                    .replace("REPLICAS", str(replicas)))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, world, port=31700 + os.getpid() % 150, env=env, timeout=400)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "COMPOSED_OK" in proc.stdout


MUON_WORKER = """
import sys, torch, torch.distributed as dist
from torch.utils.data import DataLoader, TensorDataset
from ohara_b200.models.llama import Config, Llama
from ohara_b200.runtime import EngineConfig, OharaEngine, ParallelConfig, StrategyType, TensorParallelPlan
from ohara_b200.optimizer import build_muon_adamw
from ohara_b200.trainer import Trainer
from ohara_b200.lr_scheduler import Scheduler

torch.manual_seed(0)
cfg = Config(vocab_size=32, max_sequence_length=16, hidden_size=16, intermediate_size=24,
             num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3, dropout=0.0)
ids = torch.randint(0, 32, (8, 17))
dataset = TensorDataset(ids[:, :-1], ids[:, 1:])
state = {k: v.clone() for k, v in Llama(cfg).state_dict().items()}

def solo_after(steps):
    solo = Llama(cfg); solo.load_state_dict(state)
    opt = build_muon_adamw(solo)
    for _ in range(steps):
        loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
        loss.backward(); opt.step(); opt.zero_grad()
    return solo

engine = OharaEngine(EngineConfig(
    strategy=StrategyType.FSDP, shard_parameters=True, shard_parameters_layout="matrix",
    parallel=ParallelConfig(tp=TP),
    tensor_parallel=TensorParallelPlan.llama_default(TP) if TP > 1 else TensorParallelPlan()))

def make():
    model = Llama(cfg); model.load_state_dict(state)
    model = engine.prepare(model)
    (opt,) = engine.prepare_optimizers(build_muon_adamw(model))
    dp = engine.data_parallel_world_size
    loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=8 // dp))
    trainer = Trainer(engine, model, opt, loader, loader, Scheduler(0.02), micro_batch=1,
                      max_iters=2, eval_iters=0, save_ckpt_iters=0)
    return model, opt, trainer

def close_to(model, solo):
    full = engine.full_state_dict(model)
    for name, value in solo.state_dict().items():
        assert torch.allclose(full[name], value, atol=5e-5), (name, (full[name] - value).abs().max())

model, opt, trainer = make()
assert any(group.get("kind") == "muon" for group in opt.param_groups)
trainer.train()
close_to(model, solo_after(2))
engine.save(sys.argv[1], trainer.checkpoint_state(2, 0.02, 0.0))
model, opt, trainer = make()
engine.load(sys.argv[1], {"model": model, "optimizer": opt})
trainer.train()
close_to(model, solo_after(4))
if dist.get_rank() == 0:
    print("MUON_SHARDED_OK")
engine.close()
"""


@pytest.mark.parametrize("world,tp", [(4, 1), (4, 2)])
def test_muon_on_sharded_parameters_matches_single_process_and_resumes(tmp_path, world, tp):
    """The "matrix" layout keeps whole matrices at their owners, so Muon runs there without a
    gather; the momentum buffers are checkpointed per matrix and a fresh model resumes."""
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(MUON_WORKER).replace("TP", str(tp)))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, world, port=32000 + os.getpid() % 150, env=env, timeout=400,
                        args=(str(tmp_path / "ckpt.pt"),))
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "MUON_SHARDED_OK" in proc.stdout


LOOP_MOE_WORKER = """
import torch, torch.distributed as dist
from ohara_b200.models.llama import Config, Llama
from ohara_b200.runtime import EngineConfig, OharaEngine, StrategyType
from ohara_b200.optimizer import build_adamw

torch.manual_seed(0)
cfg = Config(vocab_size=31, max_sequence_length=8, hidden_size=16, intermediate_size=24,
             num_attention_heads=2, num_hidden_layers=2, dropout=0.0, moe_num_experts=6,
             moe_experts_per_tok=1, moe_quantile_balancing=False)
ids = torch.randint(0, 31, (2, 5))                      # one short sequence per rank
state = {k: v.clone() for k, v in Llama(cfg).state_dict().items()}
solo = Llama(cfg); solo.load_state_dict(state)
ref_opt = build_adamw(solo, learning_rate=0.02, weight_decay=0.0)
engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP, shard_parameters=True))
model = Llama(cfg); model.load_state_dict(state)
model = engine.prepare(model)
(opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=0.02, weight_decay=0.0))
rank = dist.get_rank()
model.train(); solo.train()
idle = 0
for _ in range(3):
    loss = solo.loss_sum(ids[:, :-1], ids[:, 1:]) / ids[:, 1:].numel()
    loss.backward()
    for p in solo.parameters():      # a reduced gradient is zero, not absent, for an idle expert
        if p.grad is None:
            p.grad = torch.zeros_like(p)
    ref_opt.step(); ref_opt.zero_grad()
    mine = ids[rank:rank + 1]
    loss = model(mine[:, :-1], targets=mine[:, 1:]) / mine[:, 1:].numel()
    engine.backward(loss)
    opt.step(); opt.zero_grad()
from ohara_b200.modules.routing import expert_load
idle = sum(int((counts == 0).sum()) for counts in expert_load(model))
assert idle > 0, "every expert was used: the case under test did not occur"
full = engine.full_state_dict(model)
for name, value in solo.state_dict().items():
    assert torch.allclose(full[name], value, atol=3e-5), (name, (full[name] - value).abs().max())
if rank == 0:
    print("LOOP_MOE_SHARDED_OK")
engine.close()
"""


def test_experts_without_tokens_on_a_rank_do_not_desynchronise_the_reduction(tmp_path):
    """Loop MoE, one routed expert per token, four tokens per rank and six experts: on every rank
    some experts get no gradient. Their blocks are reduced at the end of the backward pass by
    every rank in turn, and training follows the single-process run."""
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(LOOP_MOE_WORKER))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    proc = launch_ranks(path, 2, port=32200 + os.getpid() % 150, env=env, timeout=400)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "LOOP_MOE_SHARDED_OK" in proc.stdout
