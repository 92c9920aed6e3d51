"""Context-parallel attention (zig-zag sharding) on two GPUs against single-device causal attention
over the whole sequence, forward and backward."""

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
    # On four or more GPUs the middle ranks run both remote passes (earlier and later owners);
    # with two ranks each rank runs one of them. OHARA_CP_TEST_RANKS overrides the count.
    default = 4 if torch.cuda.device_count() >= 4 else 2
    ranks = min(int(os.environ.get("OHARA_CP_TEST_RANKS", default)), torch.cuda.device_count())
    script = """
        import torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.ops.attention import attention_reference
        from ohara_b200.parallel.cp import CPWorkspace, context_parallel_attention, shard_sequence

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
            mine = lambda t: shard_sequence(t, rank, world)  # early block + late block of the zig-zag
            ql, kl, vl = (mine(t).clone().requires_grad_() for t in (q, k, v))
            out = context_parallel_attention(ql, kl, vl, workspace)
            out.backward(mine(upstream))
            torch.cuda.synchronize(); ops.check_status()

            qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
            ref = attention_reference(qr, kr, vr, causal=True)
            ref.backward(upstream.float())
            def close(a, b):
                return (a.float() - b.float()).abs().max().item() <= 2e-2 * (b.float().abs().max().item() + 1e-6)
            assert close(out, mine(ref)), "forward"
            assert close(ql.grad, mine(qr.grad)), "dq"
            assert close(kl.grad, mine(kr.grad)), "dk"
            assert close(vl.grad, mine(vr.grad)), "dv"
        if rank == 0:
            print("CP_OK")
        dist.destroy_process_group()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
           "--master-addr", "127.0.0.1", "--master-port", str(29800 + os.getpid() % 90), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "CP_OK" in proc.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_engine_context_parallel_llama_matches_single_device(tmp_path):
    """cp=2 through the engine: each rank runs its zig-zag half of every sequence; loss and gradients of a
    training step must match the model on whole sequences."""
    script = """
        import torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, ParallelConfig

        engine = OharaEngine(EngineConfig(parallel=ParallelConfig(cp=2)))
        engine.launch()
        rank = dist.get_rank()
        cfg = Config(vocab_size=512, max_sequence_length=512, hidden_size=256, intermediate_size=512,
                     num_attention_heads=2, num_key_value_heads=1, num_hidden_layers=2, dropout=0.0,
                     weight_tying=False)
        torch.manual_seed(0)
        reference = Llama(cfg).cuda()
        torch.manual_seed(0)
        model = engine.prepare(Llama(cfg))
        torch.manual_seed(1)
        ids = torch.randint(0, 512, (2, 513), device="cuda")
        dist.broadcast(ids, src=0)
        x, y = ids[:, :-1], ids[:, 1:]
        for step in range(2):
            xl, yl = engine.local_batch((x, y))
            assert xl.shape == (2, 256)
            with engine.autocast_context():
                loss = model(xl, targets=yl, loss_scale=1.0 / yl.numel())
            engine.backward(loss)
            engine.sync_tensor_parallel_gradients(model)  # also sums over the context-parallel group
            torch.cuda.synchronize(); ops.check_status()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                ref_loss = reference(x, targets=y, loss_scale=1.0 / y.numel())
            ref_loss.backward()
            total = loss.detach().clone() / 2
            dist.all_reduce(total)
            assert abs(float(total) - float(ref_loss)) < 2e-2 * abs(float(ref_loss)), (float(total), float(ref_loss))
            wanted = dict(reference.named_parameters())
            for name, param in model.named_parameters():
                a, b = param.grad.float(), wanted[name].grad.float()
                assert (a - b).abs().max().item() <= 6e-2 * (b.abs().max().item() + 1e-8), name
            model.zero_grad(); reference.zero_grad()
        if rank == 0:
            print("CP_ENGINE_OK")
        engine.close()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29750 + os.getpid() % 40), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "CP_ENGINE_OK" in proc.stdout
