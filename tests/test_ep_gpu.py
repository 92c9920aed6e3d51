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
