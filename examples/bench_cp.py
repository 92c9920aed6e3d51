"""Context-parallel causal attention (zig-zag sharding over NVLink peer memory), forward + backward,
against flash attention of the whole sequence on one GPU.

    torchrun --nproc-per-node 2 examples/bench_cp.py --seq 32768 --heads 16 --head-dim 128

Every rank holds ``seq / cp`` tokens (an early and a late block of the sequence). Timed on the
device with CUDA events after warm-up; the time of the step is the maximum over ranks, and the
per-rank times are printed too, since equal work per rank is the point of the zig-zag. The ideal is
the single-GPU time of the whole sequence divided by the number of ranks.
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

from ohara_b200 import ops
from ohara_b200.ops.attention import attention
from ohara_b200.parallel.cp import CPWorkspace, context_parallel_attention, shard_sequence


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
    return begin.elapsed_time(end) / steps


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--seq", type=int, default=32768, help="tokens of the whole sequence")
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--kv-heads", type=int, default=None)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    args = parser.parse_args()

    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    kv_heads = args.kv_heads or args.heads
    shape_q = (args.batch, args.seq, args.heads, args.head_dim)
    shape_kv = (args.batch, args.seq, kv_heads, args.head_dim)
    torch.manual_seed(0)
    q = torch.randn(shape_q, device="cuda").bfloat16()
    k = torch.randn(shape_kv, device="cuda").bfloat16()
    v = torch.randn(shape_kv, device="cuda").bfloat16()
    upstream = torch.randn(shape_q, device="cuda").bfloat16()

    def whole_sequence():
        qf, kf, vf = (t.detach().requires_grad_() for t in (q, k, v))
        attention(qf, kf, vf, causal=True).backward(upstream)

    single_ms = timed(whole_sequence, args.steps, args.warmup)

    local = args.seq // world
    workspace = CPWorkspace(dist.group.WORLD, local * args.batch * 2 * kv_heads * args.head_dim)
    ql, kl, vl, gl = (shard_sequence(t, rank, world).contiguous() for t in (q, k, v, upstream))

    def sharded():
        qs, ks, vs = (t.detach().requires_grad_() for t in (ql, kl, vl))
        context_parallel_attention(qs, ks, vs, workspace).backward(gl)

    mine_ms = timed(sharded, args.steps, args.warmup)
    ops.check_status()
    times = torch.zeros(world, device="cuda")
    times[rank] = mine_ms
    dist.all_reduce(times)
    single = torch.tensor([single_ms], device="cuda")
    dist.all_reduce(single, op=dist.ReduceOp.MAX)
    if rank == 0:
        step_ms = float(times.max())
        # causal attention, forward + backward: 4 * T^2 * D * H * B * 3.5 / 2 useful FLOPs
        flops = 3.5 * 4 * args.seq * args.seq * args.head_dim * args.heads * args.batch / 2
        print(json.dumps({
            "op": "context_parallel_attention_fwd_bwd", "cp": world, "seq": args.seq,
            "batch": args.batch, "heads": args.heads, "kv_heads": kv_heads,
            "head_dim": args.head_dim, "ms": step_ms,
            "per_rank_ms": [round(float(t), 3) for t in times],
            "single_gpu_whole_sequence_ms": float(single),
            "ideal_ms": float(single) / world,
            "fraction_of_ideal": float(single) / world / step_ms,
            "tflops_per_gpu": flops / world / (step_ms * 1e-3) / 1e12,
        }))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
