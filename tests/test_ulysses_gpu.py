"""Ulysses-style context parallelism on two GPUs: NCCL all-to-alls around the flash-attention
kernels must reproduce attention over the whole sequence."""

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
def test_all_to_all_attention_matches_the_whole_sequence_on_two_gpus(tmp_path):
    script = """
        import os, torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.parallel.cp import shard_sequence
        from ohara_b200.parallel.ulysses import UlyssesWorkspace, ulysses_attention
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl")
        rank, world = dist.get_rank(), dist.get_world_size()
        workspace = UlyssesWorkspace(dist.group.WORLD)
        torch.manual_seed(0)
        B, T, H, Hk, D = 2, 1024, 8, 2, 128
        q, k, v = (torch.randn(B, T, h, D, device="cuda").bfloat16() for h in (H, Hk, Hk))
        weight = torch.randn(B, T, H, D, device="cuda").bfloat16()
        mine = [shard_sequence(t, rank, world).clone().requires_grad_() for t in (q, k, v)]
        out = ulysses_attention(*mine, workspace)
        full = [t.clone().requires_grad_() for t in (q, k, v)]
        want = ops.attention(*full, causal=True)
        (out * shard_sequence(weight, rank, world)).sum().backward()
        (want * weight).sum().backward()
        torch.cuda.synchronize(); ops.check_status()
        def close(a, b):
            return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)) < 2e-2
        assert close(out, shard_sequence(want, rank, world))
        for got, ref in zip(mine, full):
            assert close(got.grad, shard_sequence(ref.grad, rank, world))
        if rank == 0:
            print("ULYSSES_GPU_OK")
        dist.destroy_process_group()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29890 + os.getpid() % 40), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "ULYSSES_GPU_OK" in proc.stdout
