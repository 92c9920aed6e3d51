"""Expert-parallel mixture of experts over peer memory on two GPUs against the same layer on one
device, forward and backward."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_layer_matches_single_device(tmp_path):
    script = """
        import os, torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.modules.moe_grouped import GroupedMoE
        from ohara_b200.parallel.ep import EPWorkspace

        dist.init_process_group("nccl")
        rank, world = dist.get_rank(), dist.get_world_size()
        torch.cuda.set_device(rank)
        torch.manual_seed(0)
        dim, hidden, experts, top_k, tokens = 256, 128, 8, 2, 384

        def make():
            torch.manual_seed(0)
            layer = GroupedMoE(dim, hidden, num_experts=experts, num_experts_per_tok=top_k,
                               num_shared_experts=1).cuda()
            with torch.no_grad():
                layer.w_down.normal_(std=0.05)
                layer.shared_down.weight.normal_(std=0.05)
            return layer.train()

        reference, sharded = make(), make()
        workspace = EPWorkspace(dist.group.WORLD, experts, capacity_rows=2048, width=dim)
        sharded.shard_experts(workspace)
        assert sharded.w_gate.shape[0] == experts // world

        # every rank routes its own tokens; the reference sees all of them
        torch.manual_seed(1)
        everything = torch.randn(world, 1, tokens, dim, device="cuda").bfloat16().float()
        upstream = torch.randn(world, 1, tokens, dim, device="cuda")
        for step in range(3):
            mine = everything[rank].clone().requires_grad_()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = sharded(mine)
            # local loss, as under data parallelism (the wrapper averages replicated gradients;
            # the expert shards scale their own)
            (out.float() * upstream[rank]).sum().backward()
            torch.cuda.synchronize(); ops.check_status()

            full = everything.clone().requires_grad_()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                ref = torch.stack([reference(full[r]) for r in range(world)])
            (ref.float() * upstream).sum().div(world).backward()

            def close(a, b, tol, rows_allowed=0.01):
                a, b = a.float().reshape(-1, a.shape[-1]), b.float().reshape(-1, b.shape[-1])
                bad = ((a - b).abs().amax(dim=1) > tol * (b.abs().max().item() + 1e-6)).float().mean().item()
                return bad <= rows_allowed
            assert close(out, ref[rank], 3e-2), "forward"
            assert close(mine.grad / world, full.grad[rank], 5e-2), "input gradient"
            local = experts // world
            for name in ("w_gate", "w_up", "w_down"):
                got = getattr(sharded, name).grad
                want = getattr(reference, name).grad[rank * local:(rank + 1) * local]
                assert close(got.flatten(1), want.flatten(1), 8e-2, 0.02), name
            # the router is replicated: its gradient is this rank's share of the reference's
            total = sharded.router.weight.grad.clone()
            dist.all_reduce(total)
            assert close(total / world, reference.router.weight.grad, 8e-2, 0.05), "router"
            reference.zero_grad(); sharded.zero_grad()
        if rank == 0:
            print("EP_OK")
        dist.destroy_process_group()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29900 + os.getpid() % 90), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "EP_OK" in proc.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_shot_all_reduce_matches_c10d(tmp_path):
    script = """
        import torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.parallel.peer import PeerRuntime

        dist.init_process_group("nccl")
        rank, world = dist.get_rank(), dist.get_world_size()
        torch.cuda.set_device(rank)
        runtime = PeerRuntime(dist.group.WORLD)
        for step, (numel, dtype) in enumerate([(1, torch.float32), (768, torch.bfloat16), (50000, torch.float32),
                                               (3, torch.bfloat16), (262144, torch.bfloat16), (4_000_000, torch.float32)]):
            torch.manual_seed(10 * step + rank)
            mine = torch.randn(numel, device="cuda").to(dtype)
            expected = mine.float().clone()
            dist.all_reduce(expected)
            got = runtime.all_reduce_(mine.clone(), average=step % 2 == 1)
            if step % 2 == 1:
                expected /= world
            torch.cuda.synchronize(); ops.check_status()
            tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
            assert torch.allclose(got.float(), expected, atol=tol, rtol=tol), (step, (got.float() - expected).abs().max())
        if rank == 0:
            print("AR_OK")
        dist.destroy_process_group()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29990 + os.getpid() % 9), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "AR_OK" in proc.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_engine_expert_parallel_llama_matches_single_device(tmp_path):
    """ep=2 through the engine (experts sharded, everything else data parallel): loss and gradients
    of a training step must match the unsharded model on the concatenated batch."""
    script = """
        import torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, ParallelConfig

        engine = OharaEngine(EngineConfig(parallel=ParallelConfig(ep=2)))
        engine.launch()
        rank, world = dist.get_rank(), dist.get_world_size()
        assert engine.data_parallel_world_size == 2 and engine.data_parallel_rank == rank
        cfg = Config(vocab_size=512, max_sequence_length=128, hidden_size=256, intermediate_size=128,
                     num_attention_heads=4, num_hidden_layers=2, dropout=0.0, weight_tying=False,
                     moe_num_experts=8, moe_experts_per_tok=2, moe_grouped=True, moe_num_shared_experts=1)
        def build():
            torch.manual_seed(0)
            model = Llama(cfg)
            with torch.no_grad():
                for block in model.layers:
                    block.ff.w_down.normal_(std=0.05)
                    block.ff.shared_down.weight.normal_(std=0.05)
            return model
        reference = build().cuda().train()
        model = engine.prepare(build()).train()
        inner = model.module
        assert inner.layers[0].ff.w_gate.shape[0] == 4

        torch.manual_seed(1)
        ids = torch.randint(0, 512, (world, 2, 129), device="cuda")
        dist.broadcast(ids, src=0)
        mine = ids[rank]
        with engine.autocast_context():
            loss = model(mine[:, :-1], targets=mine[:, 1:], loss_scale=1.0 / mine[:, 1:].numel())
        engine.backward(loss)
        engine.sync_expert_gradients(model)
        torch.cuda.synchronize(); ops.check_status()
        everything = ids.view(-1, 129)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            ref_loss = reference(everything[:, :-1], targets=everything[:, 1:],
                                 loss_scale=1.0 / everything[:, 1:].numel())
        ref_loss.backward()
        total = loss.detach().clone()
        dist.all_reduce(total)
        assert abs(float(total) / world - float(ref_loss)) < 2e-2 * abs(float(ref_loss))
        wanted = dict(reference.named_parameters())
        def close(a, b, tol, rows_allowed=0.02):
            a, b = a.float().reshape(-1, a.shape[-1]), b.float().reshape(-1, b.shape[-1])
            bad = ((a - b).abs().amax(dim=1) > tol * (b.abs().max().item() + 1e-8)).float().mean().item()
            return bad <= rows_allowed
        for name, param in inner.named_parameters():
            want = wanted[name].grad
            if getattr(param, "expert_parallel", False):
                want = want[rank * 4:(rank + 1) * 4]
            assert close(param.grad, want, 8e-2), name
        if rank == 0:
            print("EP_ENGINE_OK")
        engine.close()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29850 + os.getpid() % 40), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "EP_ENGINE_OK" in proc.stdout
