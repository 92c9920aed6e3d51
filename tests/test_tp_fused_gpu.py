"""Tensor-parallel linears with the collectives fused into the GEMM (all-gather -> GEMM through peer
TMA loads, GEMM -> reduce-scatter through peer stores) against a single-device fp32 reference, on two
GPUs; plus a one-GPU check that a missing peer flag ends the fused GEMM with a status, not a hang."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_gather_gemm_gives_up_when_a_peer_never_signals():
    """World of 2 emulated on one device: rank 1's ready flag is never written. The producer's wait
    must run out, the kernel must unwind (TMEM freed) and the context must stay usable."""
    from ohara_b200 import ops
    from ohara_b200.ops._ext import ext

    C = ext()
    C.status(True)
    rows, width, features = 128, 256, 256
    mine = torch.randn(rows, width, device="cuda").bfloat16()
    other = torch.randn(rows, width, device="cuda").bfloat16()
    weight = torch.randn(features, width, device="cuda").bfloat16()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    maps = C.peer_row_maps([mine.data_ptr(), other.data_ptr()], rows, width, width, 0)
    out = torch.zeros(2 * rows, features, device="cuda", dtype=torch.bfloat16)
    C.gemm_gather_a(maps, mine, weight, out, False, flags.data_ptr(), 1, 0, 2, 0.2)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="peer flag"):
        ops.check_status()
    # once the flag is there the same call completes and is correct for both row blocks
    flags[1] = 1
    C.gemm_gather_a(maps, mine, weight, out, False, flags.data_ptr(), 1, 0, 2, 0.2)
    torch.cuda.synchronize()
    ops.check_status()
    ref = torch.cat([mine, other]).float() @ weight.float().t()
    assert (out.float() - ref).abs().max() <= 1e-2 * ref.abs().max()


def test_push_epilogue_and_slot_reduction_on_one_device():
    """Both 'ranks' of a reduce-scatter emulated one after the other on one device."""
    from ohara_b200 import ops
    from ohara_b200.ops._ext import ext

    C = ext()
    C.status(True)
    rows, width, features, world = 256, 320, 192, 2
    block = rows // world
    a = [torch.randn(rows, width, device="cuda").bfloat16() for _ in range(world)]
    w = [torch.randn(features, width, device="cuda").bfloat16() for _ in range(world)]
    receive = [torch.zeros(world, block, features, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    slot_bytes = block * features * 2
    for rank in range(world):
        destinations = [receive[owner].data_ptr() + rank * slot_bytes for owner in range(world)]
        C.gemm_push_c(a[rank], w[rank], False, destinations, features, features, rank)
        C.tp_signal([flags.data_ptr(), flags.data_ptr()], 16, rank, 1)
    total = sum(x.float() @ y.float().t() for x, y in zip(a, w))
    for owner in range(world):
        out = C.tp_reduce_slots(receive[owner], flags.data_ptr() + 64, None, 1, 0.2)
        ref = total[owner * block : (owner + 1) * block]
        assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    torch.cuda.synchronize()
    ops.check_status()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_tensor_parallel_mlp_matches_single_device(tmp_path):
    script = """
        import os, torch, torch.distributed as dist
        import torch.nn as nn
        from ohara_b200 import ops
        from ohara_b200.parallel.tp_fused import TPWorkspace
        from ohara_b200.runtime.enums import TensorParallelStyle
        from ohara_b200.runtime.tensor_parallel import (TensorParallelPlan, TensorParallelRule,
            apply_tensor_parallel, attach_fused_workspace)

        dist.init_process_group("nccl")
        rank, world = dist.get_rank(), dist.get_world_size()
        torch.cuda.set_device(rank)
        torch.manual_seed(0)
        d, h, batch, seq = 256, 512, 4, 128

        class MLP(nn.Module):
            def __init__(self):
                super().__init__()
                self.up, self.gate, self.down = nn.Linear(d, h, bias=False), nn.Linear(d, h, bias=False), nn.Linear(h, d, bias=False)
            def forward(self, x):
                return self.down(ops.swiglu(self.gate(x), self.up(x)))

        reference = MLP().cuda()
        plan = TensorParallelPlan(degree=world, sequence_parallel=True, rules=[
            TensorParallelRule("up", TensorParallelStyle.COLWISE), TensorParallelRule("gate", TensorParallelStyle.COLWISE),
            TensorParallelRule("down", TensorParallelStyle.ROWWISE)])
        sharded = MLP().cuda()
        sharded.load_state_dict(reference.state_dict())
        apply_tensor_parallel(sharded, dist.group.WORLD, plan)
        workspace = TPWorkspace(dist.group.WORLD, rows_local=batch // world * seq, width=max(d, h))
        assert attach_fused_workspace(sharded, workspace) == 3

        x = torch.randn(batch, seq, d, device="cuda")
        dist.broadcast(x, src=0)
        upstream = torch.randn(batch, seq, d, device="cuda")
        dist.broadcast(upstream, src=0)
        per = batch // world
        for step in range(3):  # several rounds: buffers are recycled
            xr = x.clone().requires_grad_()
            (reference(xr) * upstream).sum().backward()
            xs = x[rank * per:(rank + 1) * per].clone().requires_grad_()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                ys = sharded(xs)
            assert ys.shape == (per, seq, d)
            (ys.float() * upstream[rank * per:(rank + 1) * per]).sum().backward()
            torch.cuda.synchronize(); ops.check_status()
            with torch.no_grad():
                yr = reference(x)
            def close(a, b, tol):
                return (a.float() - b.float()).abs().max().item() <= tol * (b.float().abs().max().item() + 1e-6)
            assert close(ys, yr[rank * per:(rank + 1) * per], 3e-2), "forward"
            assert close(xs.grad, xr.grad[rank * per:(rank + 1) * per], 4e-2), "input gradient"
            for name in ("up", "gate"):
                full = getattr(reference, name).weight.grad
                mine = getattr(sharded, name).weight.grad
                assert close(mine, full.chunk(world, dim=0)[rank], 4e-2), name
            assert close(sharded.down.weight.grad, reference.down.weight.grad.chunk(world, dim=1)[rank], 4e-2), "down"
            reference.zero_grad(); sharded.zero_grad()
        if rank == 0:
            print("TP_FUSED_OK")
        dist.destroy_process_group()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "TP_FUSED_OK" in proc.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_engine_sequence_parallel_llama_matches_single_device(tmp_path):
    """A Llama prepared by the engine with tp=2 and the sequence-parallel plan (fused collectives)
    must produce the loss and the gradients of the unsharded model on the whole batch."""
    script = """
        import torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, ParallelConfig, TensorParallelPlan

        engine = OharaEngine(EngineConfig(parallel=ParallelConfig(tp=2),
                                          tensor_parallel=TensorParallelPlan.llama_default(2, True)))
        engine.launch()
        rank = dist.get_rank()
        cfg = Config(vocab_size=512, max_sequence_length=128, hidden_size=256, intermediate_size=512,
                     num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, dropout=0.0,
                     weight_tying=False)
        torch.manual_seed(0)
        reference = Llama(cfg).cuda()
        torch.manual_seed(0)
        model = engine.prepare(Llama(cfg))
        assert getattr(engine, "_tp_batch_sharding", False)

        torch.manual_seed(1)
        ids = torch.randint(0, 512, (4, 129), device="cuda")
        dist.broadcast(ids, src=0)
        x, y = ids[:, :-1], ids[:, 1:]
        for step in range(2):
            xl, yl = engine.local_batch((x, y))
            assert xl.shape[0] == 2
            with engine.autocast_context():
                loss = model(xl, targets=yl, loss_scale=1.0 / yl.numel())
            engine.backward(loss)
            engine.sync_tensor_parallel_gradients(model)
            torch.cuda.synchronize(); ops.check_status()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                ref_loss = reference(x, targets=y, loss_scale=1.0 / y.numel())
            ref_loss.backward()
            total = loss.detach().clone() / 2
            dist.all_reduce(total)
            assert abs(float(total) - float(ref_loss)) < 2e-2 * abs(float(ref_loss)), (float(total), float(ref_loss))

            full = engine.full_state_dict(model)
            for key, value in reference.state_dict().items():
                assert torch.equal(full[key].cpu(), value.cpu()), key
            ref_grads = dict(reference.named_parameters())
            def close(a, b, tol=6e-2):
                return (a.float() - b.float()).abs().max().item() <= tol * (b.float().abs().max().item() + 1e-8)
            for name, param in model.named_parameters():
                want = ref_grads[name].grad
                dim = getattr(param, "tensor_parallel_dim", None)
                if dim is not None:
                    want = want.chunk(2, dim=dim)[rank]
                assert close(param.grad, want), name
            model.zero_grad(); reference.zero_grad()
        if rank == 0:
            print("SP_LLAMA_OK")
        engine.close()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + os.getpid() % 90), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "SP_LLAMA_OK" in proc.stdout
