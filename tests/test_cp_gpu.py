"""Context-parallel attention on two GPUs against single-device causal attention over the whole
sequence, forward and backward."""

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
def test_context_parallel_attention_matches_full_sequence(tmp_path):
    script = """
        import torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.ops.attention import attention_reference
        from ohara_b200.parallel.cp import CPWorkspace, context_parallel_attention

        dist.init_process_group("nccl")
        rank, world = dist.get_rank(), dist.get_world_size()
        torch.cuda.set_device(rank)
        batch, chunk, heads, kv_heads, dim = 2, 256, 4, 2, 128
        workspace = CPWorkspace(dist.group.WORLD, chunk * batch * 2 * kv_heads * dim)
        for step in range(3):
            torch.manual_seed(step)
            q = torch.randn(batch, world * chunk, heads, dim, device="cuda").bfloat16()
            k = torch.randn(batch, world * chunk, kv_heads, dim, device="cuda").bfloat16()
            v = torch.randn(batch, world * chunk, kv_heads, dim, device="cuda").bfloat16()
            upstream = torch.randn(batch, world * chunk, heads, dim, device="cuda").bfloat16()
            rows = slice(rank * chunk, (rank + 1) * chunk)
            ql, kl, vl = (t[:, rows].clone().requires_grad_() for t in (q, k, v))
            out = context_parallel_attention(ql, kl, vl, workspace)
            out.backward(upstream[:, rows])
            torch.cuda.synchronize(); ops.check_status()

            qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
            ref = attention_reference(qr, kr, vr, causal=True)
            ref.backward(upstream.float())
            def close(a, b):
                return (a.float() - b.float()).abs().max().item() <= 2e-2 * (b.float().abs().max().item() + 1e-6)
            assert close(out, ref[:, rows]), "forward"
            assert close(ql.grad, qr.grad[:, rows]), "dq"
            assert close(kl.grad, kr.grad[:, rows]), "dk"
            assert close(vl.grad, vr.grad[:, rows]), "dv"
        if rank == 0:
            print("CP_OK")
        dist.destroy_process_group()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29800 + os.getpid() % 90), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "CP_OK" in proc.stdout
