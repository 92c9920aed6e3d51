"""Peer-memory runtime on the GPU: bounded barrier wait (1 GPU) and the fused sharded step on
two GPUs against the c10d path."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_barrier_wait_runs_out_and_reports_status():
    """A flag that nothing sets: the wait must end by itself, record a status, and leave the
    context usable."""
    from ohara_b200 import ops
    from ohara_b200.ops._ext import ext

    C = ext()
    C.status(True)
    pad_a = torch.zeros(1024, dtype=torch.int32, device="cuda")
    pad_b = torch.zeros(1024, dtype=torch.int32, device="cuda")
    # "world" of 2 emulated on one device: rank 0's own pad is pad_a; slot 1 is never written.
    C.peer_barrier([pad_a.data_ptr(), pad_b.data_ptr()], 0, 1, 0.25)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="peer flag"):
        ops.check_status()
    assert int(pad_b[0]) == 1  # our own signal did reach the "peer"
    # a satisfied barrier passes: pre-set the missing flag
    pad_a[1] = 2
    C.peer_barrier([pad_a.data_ptr(), pad_b.data_ptr()], 0, 2, 0.25)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_released_stream_wait_lets_the_streams_drain():
    """A copy stream parked in a stream-ordered wait on a flag that nothing sets (a lost peer)
    must be freed by ``release_stream_waits``: afterwards the work queued behind the wait runs
    and ``synchronize`` returns."""
    import time

    from ohara_b200.ops._ext import ext
    from ohara_b200.parallel.peer import release_stream_waits

    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    payload = torch.zeros(1024, device="cuda")
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ext().stream_wait_value32(flags.data_ptr() + 4 * 3, 7)   # epoch 7 of peer 3: never written
        payload.add_(1.0)                                         # queued behind the wait
    time.sleep(0.2)
    assert not side.query()                                       # parked, as expected
    release_stream_waits([flags.data_ptr() + 4 * r for r in range(8)])
    deadline = time.monotonic() + 10
    while not side.query() and time.monotonic() < deadline:
        time.sleep(0.01)
    drained = side.query()
    if not drained:                                               # second way out before failing
        flags.fill_(0x7FFFFFFF)
    torch.cuda.synchronize()
    assert drained, "the stream-ordered wait was not released"
    assert float(payload.sum()) == 1024.0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_sharded_step_matches_c10d_on_two_gpus(tmp_path):
    script = """
        import os, torch, torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, StrategyType
        from ohara_b200.optimizer import build_adamw, build_muon_adamw
        from ohara_b200 import ops
        # Adam-type updates are sign-like for tiny gradients, so whole-training comparisons are
        # ill-conditioned; compare the collectives themselves and a small-lr AdamW step instead.
        reduced, params, flats = {}, {}, {}
        for fused in (False, True):
            torch.manual_seed(0)
            engine = OharaEngine(EngineConfig(strategy=StrategyType.FSDP, fused_collectives=fused))
            engine.launch()
            cfg = Config(vocab_size=512, max_sequence_length=128, hidden_size=256,
                         intermediate_size=512, num_attention_heads=2, num_hidden_layers=2, dropout=0.0)
            model = engine.prepare(Llama(cfg))
            (opt,) = engine.prepare_optimizers(build_adamw(model, learning_rate=1e-3, weight_decay=0.1))
            assert opt.fused == fused, (opt.fused, fused)
            (muon,) = engine.prepare_optimizers(build_muon_adamw(model))
            assert muon.fused == fused and muon.matrix_size > 0
            gen = torch.Generator().manual_seed(5 + dist.get_rank())
            for step in range(2):
                ids = torch.randint(0, 512, (4, 129), generator=gen).cuda()
                with engine.autocast_context():
                    loss = model(ids[:, :-1], targets=ids[:, 1:], loss_scale=1.0 / (4 * 128))
                loss.backward()
                if step == 1:
                    muon.reduce_gradients()
                    reduced[fused] = (opt.reduce_gradients(), opt.grad_local.clone(),
                                      muon.grad_local.clone())
                opt.step(); opt.zero_grad()
                muon._reduced = False
            torch.cuda.synchronize(); ops.check_status()
            params[fused] = [p.detach().float().clone() for p in model.parameters()]
            flats[fused] = opt.weight_flat.float().clone()
            # every rank must hold the same gathered weights
            mine = opt.weight_flat.float().clone()
            other = mine.clone(); dist.broadcast(other, src=0)
            assert torch.equal(mine, other)
        for idx in (1, 2):
            a, b = reduced[False][idx], reduced[True][idx]
            scale = a.abs().max().item() + 1e-12
            assert (a - b).abs().max().item() / scale < 2e-2, (idx, (a - b).abs().max(), scale)
        for a, b in zip(params[False], params[True]):
            assert torch.allclose(a, b, atol=6e-3), (a - b).abs().max()  # 2 steps x 2 x lr for sign flips
        if dist.get_rank() == 0:
            print("PEER_OK")
        dist.destroy_process_group()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29300 + os.getpid() % 300), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "PEER_OK" in proc.stdout
