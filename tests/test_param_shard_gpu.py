"""Parameter sharding on the GPU kernels: the gathered fp32 parameters feed the bf16 compute
copies, which must be rebuilt whenever a unit lands in a new buffer."""

import copy
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

from ohara_b200 import Config, Llama, ops
from ohara_b200.optimizer import build_adamw
from ohara_b200.parallel.param_shard import ParameterShardedOptimizer, shard_llama

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _losses(model, optimizer, batches, finish=None):
    losses = []
    for tokens in batches:
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(tokens[:, :-1], targets=tokens[:, 1:]) / tokens[:, 1:].numel()
        loss.backward()
        if finish is not None:
            finish()
        optimizer.step()
        optimizer.zero_grad()
        losses.append(float(loss.detach()))
    return losses


@pytest.mark.parametrize("checkpoint", [False, True])
def test_sharded_model_on_one_gpu_follows_the_plain_model(checkpoint):
    torch.manual_seed(0)
    cfg = Config(vocab_size=512, max_sequence_length=256, hidden_size=256, intermediate_size=384,
                 num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3, dropout=0.0)
    plain = Llama(cfg).cuda()
    sharded = copy.deepcopy(plain)
    if checkpoint:
        sharded.enable_activation_checkpointing()
    sharding = shard_llama(sharded)
    plain_opt = build_adamw(plain, learning_rate=3e-3, weight_decay=0.1)
    sharded_opt = ParameterShardedOptimizer(
        build_adamw(sharded, learning_rate=3e-3, weight_decay=0.1), sharding)
    plain.train(), sharded.train()
    batches = [torch.randint(0, 512, (4, 193), device="cuda")] * 5   # one batch, seen five times
    want = _losses(plain, plain_opt, batches)
    got = _losses(sharded, sharded_opt, batches, finish=sharding.finish_backward)
    torch.cuda.synchronize()
    ops.check_status()
    # same kernels on the same values: the curves agree to the order of the bf16 rounding of
    # the refreshed weights (a stale compute copy would leave the loss where it started)
    assert got == pytest.approx(want, rel=2e-3)
    assert got[-1] < got[0] - 0.05
    assert all(u.full is None for u in sharding.units)
    full = sharding.full_state_dict(sharded)
    for name, value in plain.state_dict().items():
        assert torch.allclose(full[name], value, atol=2e-3), name


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_match_single_device_training(tmp_path):
    script = """
        import torch, torch.distributed as dist
        from torch.utils.data import DataLoader, TensorDataset
        from ohara_b200 import ops
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, StrategyType
        from ohara_b200.optimizer import build_adamw
        from ohara_b200.trainer import Trainer
        from ohara_b200.lr_scheduler import Scheduler

        torch.manual_seed(0)
        cfg = Config(vocab_size=512, max_sequence_length=128, hidden_size=256, intermediate_size=384,
                     num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3, dropout=0.0)
        ids = torch.randint(0, 512, (8, 129))
        dataset = TensorDataset(ids[:, :-1], ids[:, 1:])
        state = {k: v.clone() for k, v in Llama(cfg).state_dict().items()}
        engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP, shard_parameters=True))
        engine.launch()

        solo = Llama(cfg); solo.load_state_dict(state); solo = solo.to(engine.device)
        ref_opt = build_adamw(solo, learning_rate=3e-3, weight_decay=0.1)
        want = []
        for _ in range(5):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = solo.loss_sum(ids[:, :-1].to(engine.device), ids[:, 1:].to(engine.device)) / ids[:, 1:].numel()
            loss.backward(); ref_opt.step(); ref_opt.zero_grad(); want.append(float(loss.detach()))

        model = Llama(cfg); model.load_state_dict(state)
        model = engine.prepare(model)
        (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=3e-3, weight_decay=0.1))
        loader = engine.prepare_dataloaders(DataLoader(dataset, batch_size=4))
        trainer = Trainer(engine, model, opt, loader, loader, Scheduler(3e-3), micro_batch=1,
                          max_iters=5, eval_iters=0, save_ckpt_iters=0)
        got = []
        for step in range(1, 6):
            loss, _ = trainer.train_step(step)
            total = torch.tensor([loss], device=engine.device)
            dist.all_reduce(total)
            got.append(float(total) / dist.get_world_size())
        torch.cuda.synchronize(); ops.check_status()
        assert all(abs(a - b) < 3e-3 * abs(b) for a, b in zip(got, want)), (got, want)
        report = model._param_sharding.memory_report()
        assert report["persistent_bytes_per_rank"] < 0.6 * report["unsharded_bytes"]
        if dist.get_rank() == 0:
            print("PARAM_SHARD_GPU_OK", report)
        engine.close()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29950 + os.getpid() % 40), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "PARAM_SHARD_GPU_OK" in proc.stdout
