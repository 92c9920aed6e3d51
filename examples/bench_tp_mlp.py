"""Tensor-parallel SwiGLU MLP block (sequence-parallel layout), forward + backward: the collectives
fused into the GEMM over NVLink peer memory against the same layers on c10d (NCCL) collectives.

    torchrun --nproc-per-node 4 examples/bench_tp_mlp.py --hidden 2048 --ffn 5632 --tokens 8192

Each rank holds ``tokens / tp`` rows between the parallel regions. Timed on the device with CUDA
events after warm-up, maximum over ranks. The roofline printed for the fused path is the slower of
(FLOPs / measured bf16 GEMM rate) and (bytes that must cross NVLink per GPU / 770 GB/s).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist
import torch.nn as nn

from ohara_b200 import ops
from ohara_b200.parallel.tp_fused import TPWorkspace
from ohara_b200.runtime.enums import TensorParallelStyle
from ohara_b200.runtime.tensor_parallel import (
    TensorParallelPlan,
    TensorParallelRule,
    apply_tensor_parallel,
    attach_fused_workspace,
)
from ohara_b200.trainer import measured_peak_flops


class MLP(nn.Module):
    def __init__(self, hidden: int, ffn: int) -> None:
        super().__init__()
        self.gate = nn.Linear(hidden, ffn, bias=False)
        self.up = nn.Linear(hidden, ffn, bias=False)
        self.down = nn.Linear(ffn, hidden, bias=False)

    def forward(self, x):
        return self.down(ops.swiglu(self.gate(x), self.up(x)))


def timed(fn, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        fn()
    end.record()
    end.synchronize()
    elapsed = torch.tensor([begin.elapsed_time(end) / steps], device="cuda")
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    return float(elapsed)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--ffn", type=int, default=5632)
    p.add_argument("--tokens", type=int, default=8192, help="tokens per tensor-parallel group")
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    args = p.parse_args()

    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    torch.manual_seed(0)
    rows_local = args.tokens // world
    plan = TensorParallelPlan(degree=world, sequence_parallel=True, rules=[
        TensorParallelRule("gate", TensorParallelStyle.COLWISE),
        TensorParallelRule("up", TensorParallelStyle.COLWISE),
        TensorParallelRule("down", TensorParallelStyle.ROWWISE)])
    results = {}
    for fused in (False, True):
        model = apply_tensor_parallel(MLP(args.hidden, args.ffn).cuda(), dist.group.WORLD, plan)
        if fused:
            workspace = TPWorkspace(dist.group.WORLD, rows_local, max(args.hidden, args.ffn // world))
            attach_fused_workspace(model, workspace)
            x = torch.randn(1, rows_local, args.hidden, device="cuda", dtype=torch.bfloat16)
        else:
            x = torch.randn(1, rows_local, args.hidden, device="cuda", dtype=torch.bfloat16)
        x.requires_grad_()
        upstream = torch.randn(1, rows_local, args.hidden, device="cuda", dtype=torch.bfloat16)

        def step():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = model(x)
            y.backward(upstream)
            model.zero_grad(set_to_none=True)
            x.grad = None

        results["fused" if fused else "c10d"] = timed(step, args.steps, args.warmup)
        torch.cuda.synchronize()
        ops.check_status()

    flops = 6.0 * args.tokens * args.hidden * (args.ffn // world) * 3  # fwd + dgrad + wgrad, 3 matrices
    peak = measured_peak_flops() or 1.4e15
    # Per GPU and direction: 2 gathers + 1 scatter forward, 2 scatters + 1 gather (+3 for the weight
    # gradients' operands) backward, each moving (world - 1) / world of a tokens x hidden bf16 matrix.
    moved = 9 * (world - 1) / world * args.tokens * args.hidden * 2
    roofline_ms = max(flops / peak, moved / 770e9) * 1e3
    if rank == 0:
        print(json.dumps({
            "bench": "tp_mlp_fwd_bwd", "tp": world, "hidden": args.hidden, "ffn": args.ffn,
            "tokens": args.tokens, "c10d_ms": results["c10d"], "fused_ms": results["fused"],
            "speedup": results["c10d"] / results["fused"], "roofline_ms": roofline_ms,
            "fused_fraction_of_roofline": roofline_ms / results["fused"],
            "compute_ms": flops / peak * 1e3, "nvlink_ms": moved / 770e9 * 1e3,
        }))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
