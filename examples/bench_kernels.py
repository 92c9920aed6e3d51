"""Micro-benchmarks of the hand-written kernels against their library counterparts on one GPU.

    python examples/bench_kernels.py                       # every operation, one JSON line each
    python examples/bench_kernels.py --op gemm_nt --m 65536 --n 768 --k 768
    python examples/bench_kernels.py --op attn_fwd --no-baseline --iters 3    # for a profiler

Timing: CUDA events on the launching stream after warm-up; a buffer larger than L2 is written
between iterations so that no iteration finds its inputs cached. ``fraction_of_measured`` divides
the achieved rate by the machine's measured peak (``MEASURED_PEAKS.json`` when present): the bf16
GEMM burst rate for tensor-core kernels, the copy bandwidth for bandwidth kernels.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import torch
import torch.nn.functional as F

from ohara_b200 import ops


def peaks() -> tuple[float, float]:
    try:
        data = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(data["bf16_tflops"]) * 1e12, float(data["hbm_gbs"]) * 1e9
    except (OSError, KeyError, ValueError):
        return 1.59e15, 6.65e12


class Timer:
    def __init__(self, iters: int, warmup: int) -> None:
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        total = 0.0
        for _ in range(self.iters):
            self.flush.zero_()  # evict L2
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            fn()
            end.record()
            end.synchronize()
            total += begin.elapsed_time(end)
        return total / self.iters / 1e3


def bf(*shape):
    return torch.randn(*shape, device="cuda").bfloat16()


def bench_gemm(kind, args, timer):
    m, n, k = args.m, args.n, args.k
    if kind == "gemm_nt":
        a, b = bf(m, k), bf(n, k)
        ours, base = (lambda: ops.matmul_nt(a, b)), (lambda: a @ b.t())
    elif kind == "gemm_nn":
        a, b = bf(m, k), bf(k, n)
        ours, base = (lambda: ops.matmul_nn(a, b)), (lambda: a @ b)
    else:  # weight gradient: (K, M)^T @ (K, N) in fp32
        a, b = bf(k, m), bf(k, n)
        ours = lambda: ops.matmul_tn(a, b)  # noqa: E731
        base = lambda: torch.mm(a.t(), b, out_dtype=torch.float32) if False else (a.t() @ b).float()  # noqa: E731
    return dict(shape=[m, n, k], work=2.0 * m * n * k, kind="flops", ours=ours, baseline=base)


def bench_attention(kind, args, timer):
    b, t, h, hk, d = args.batch, args.seq, args.heads, args.kv_heads or args.heads, args.head_dim
    q, k, v = bf(b, t, h, d), bf(b, t, hk, d), bf(b, t, hk, d)
    flops = 4.0 * b * h * t * t * d / 2  # causal
    if kind == "attn_fwd":
        ours = lambda: ops.attention(q, k, v, causal=True)  # noqa: E731
        qs, ks, vs = (x.transpose(1, 2) for x in (q, k, v))
        base = lambda: F.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=h != hk)  # noqa: E731
        return dict(shape=[b, t, h, hk, d], work=flops, kind="flops", ours=ours, baseline=base)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    out = ops.attention(q, k, v, causal=True)
    grad = torch.randn_like(out)
    ours = lambda: torch.autograd.grad(out, (q, k, v), grad, retain_graph=True)  # noqa: E731
    qs, ks, vs = (x.detach().transpose(1, 2).requires_grad_() for x in (q, k, v))
    ref = F.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=h != hk)
    gref = grad.transpose(1, 2)
    base = lambda: torch.autograd.grad(ref, (qs, ks, vs), gref, retain_graph=True)  # noqa: E731
    return dict(shape=[b, t, h, hk, d], work=2.5 * flops, kind="flops", ours=ours, baseline=base)


def bench_bandwidth(kind, args, timer):
    rows, d = args.m, args.n
    x = bf(rows, d)
    if kind == "rmsnorm":
        w = torch.ones(d, device="cuda")
        ours = lambda: ops.rms_norm(x, w)  # noqa: E731
        base = lambda: F.rms_norm(x.float(), (d,), w, 1e-5).bfloat16()  # noqa: E731
        moved = 2.0 * rows * d * 2
    elif kind == "swiglu":
        y = bf(rows, d)
        ours = lambda: ops.swiglu(x, y)  # noqa: E731
        base = lambda: F.silu(x) * y  # noqa: E731
        moved = 3.0 * rows * d * 2
    else:  # cross_entropy rows kernel through the fused loss
        vocab = args.k
        hidden, weight = bf(rows, d), bf(vocab, d)
        target = torch.randint(0, vocab, (rows,), device="cuda")
        ours = lambda: ops.linear_cross_entropy(hidden, weight, target, -1, 1.0)  # noqa: E731
        base = lambda: F.cross_entropy((hidden @ weight.t()).float(), target, reduction="sum")  # noqa: E731
        return dict(shape=[rows, d, vocab], work=2.0 * rows * d * vocab, kind="flops", ours=ours,
                    baseline=base)
    return dict(shape=[rows, d], work=moved, kind="bytes", ours=ours, baseline=base)


OPS = {
    "gemm_nt": bench_gemm, "gemm_nn": bench_gemm, "gemm_tn": bench_gemm,
    "attn_fwd": bench_attention, "attn_bwd": bench_attention,
    "rmsnorm": bench_bandwidth, "swiglu": bench_bandwidth, "linear_ce": bench_bandwidth,
}
DEFAULTS = {
    "gemm_nt": dict(m=65536, n=768, k=768), "gemm_nn": dict(m=65536, n=768, k=2048),
    "gemm_tn": dict(m=768, n=2048, k=65536), "rmsnorm": dict(m=65536, n=768),
    "swiglu": dict(m=65536, n=2048), "linear_ce": dict(m=8192, n=768, k=50304),
}


def main() -> None:
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--op", choices=["all", *OPS], default="all")
    p.add_argument("--m", type=int, default=None)
    p.add_argument("--n", type=int, default=None)
    p.add_argument("--k", type=int, default=None)
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--seq", type=int, default=2048)
    p.add_argument("--heads", type=int, default=6)
    p.add_argument("--kv-heads", type=int, default=0)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--no-baseline", action="store_true")
    args = p.parse_args()
    flop_peak, byte_peak = peaks()
    timer = Timer(args.iters, args.warmup)
    for name in (OPS if args.op == "all" else [args.op]):
        local = argparse.Namespace(**vars(args))
        for key, value in DEFAULTS.get(name, {}).items():
            if getattr(local, key) is None:
                setattr(local, key, value)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            case = OPS[name](name, local, timer)
            seconds = timer(case["ours"])
            baseline = None if args.no_baseline else timer(case["baseline"])
        peak = flop_peak if case["kind"] == "flops" else byte_peak
        rate = case["work"] / seconds
        line = {"op": name, "shape": case["shape"], "ms": seconds * 1e3,
                ("tflops" if case["kind"] == "flops" else "gbs"): rate / (1e12 if case["kind"] == "flops" else 1e9),
                "fraction_of_measured": rate / peak}
        if baseline is not None:
            line["library_ms"] = baseline * 1e3
            line["speedup_vs_library"] = baseline / seconds
        print(json.dumps(line), flush=True)
    ops.check_status()


if __name__ == "__main__":
    main()
