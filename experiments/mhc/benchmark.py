"""Times the Sinkhorn projection of manifold hyper-connections, forward and backward: the CUDA
kernels of ``ohara_b200.ops.sinkhorn`` against the PyTorch expression of the same iterations
(reference: experiments/mHC/benchmark.py:141-245, which compares its Triton kernel with eager).

    python experiments/mhc/benchmark.py --sizes 4,8,16,32,64 --matrices 65536 --iters 20

CUDA events around ``--repeat`` calls after ``--warmup`` untimed ones; prints one line per size
with both times, the ratio and the largest difference between the two results."""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from ohara_b200.ops.sinkhorn import sinkhorn_log, sinkhorn_reference  # noqa: E402


def _time(fn, warmup: int, repeat: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeat):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / repeat


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--sizes", default="4,8,16,32,64")
    parser.add_argument("--matrices", type=int, default=65536)
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--repeat", type=int, default=10)
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark needs a CUDA device")
    for n in (int(s) for s in args.sizes.split(",")):
        count = max(1, args.matrices * 16 // (n * n))  # the same number of elements per size
        logits = torch.randn(count, n, n, device="cuda", requires_grad=True)
        upstream = torch.randn(count, n, n, device="cuda")

        def run(fn):
            logits.grad = None
            fn(logits, args.iters).backward(upstream)

        ours = _time(lambda: run(sinkhorn_log), args.warmup, args.repeat)
        eager = _time(lambda: run(sinkhorn_reference), args.warmup, args.repeat)
        with torch.no_grad():
            gap = (sinkhorn_log(logits, args.iters) - sinkhorn_reference(logits, args.iters)).abs().max()
        print(f"n={n:3d} matrices={count:7d} kernels {ours:8.3f} ms  eager {eager:8.3f} ms  "
              f"x{eager / ours:6.2f}  max |difference| {float(gap):.2e}")


if __name__ == "__main__":
    main()
