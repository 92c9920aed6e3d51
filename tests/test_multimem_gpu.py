"""All-reduce through NVSwitch multicast (``multimem.ld_reduce``) on two GPUs against the sum
computed from the gathered inputs."""

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
@pytest.mark.skipif(os.environ.get("OHARA_TEST_MULTICAST") != "1",
                    reason="binds GPU memory to an NVLink multicast object: run it on its own, "
                           "with OHARA_TEST_MULTICAST=1, not inside a blanket test run")
def test_multicast_all_reduce_matches_the_sum_of_the_gathered_inputs(tmp_path):
    script = """
        import os, torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.parallel.multimem import MulticastAllReduce
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl")
        rank, world = dist.get_rank(), dist.get_world_size()
        try:
            reducer = MulticastAllReduce(dist.group.WORLD, max_bytes=1 << 18, wait_limit_s=5.0)
        except RuntimeError as error:
            if rank == 0:
                print("MULTICAST_UNSUPPORTED", error)
            dist.destroy_process_group()
            raise SystemExit(0)
        torch.manual_seed(rank)
        for step, (dtype, count) in enumerate([(torch.float32, 4), (torch.bfloat16, 8),
                                               (torch.float32, 4096), (torch.bfloat16, 6144),
                                               (torch.bfloat16, 1 << 17), (torch.float32, 1 << 16)]):
            mine = torch.randn(count, device="cuda").to(dtype)
            everyone = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(everyone, mine)
            want = torch.stack([t.float() for t in everyone]).sum(0)
            average = step % 2 == 1
            got = reducer.all_reduce_(mine.clone(), average=average).float()
            if average:
                want = want / world
            torch.cuda.synchronize(); ops.check_status()
            tolerance = 1e-6 if dtype == torch.float32 else 1e-2
            assert torch.allclose(got, want, rtol=tolerance, atol=tolerance), (dtype, count)
        reducer.close()
        if rank == 0:
            print("MULTICAST_OK")
        dist.destroy_process_group()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29940 + os.getpid() % 40), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    if "MULTICAST_UNSUPPORTED" in proc.stdout:
        pytest.skip("no NVLink multicast on this machine")
    assert "MULTICAST_OK" in proc.stdout
