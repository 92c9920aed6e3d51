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
        if kind == "linear_ce_train":
            # training form: the fused op also produces both gradients in its forward pass; the
            # library arm runs forward + backward
            hidden.requires_grad_()
            weight.requires_grad_()

            def library():
                hidden.grad = weight.grad = None
                F.cross_entropy((hidden @ weight.t()).float(), target, reduction="sum").backward()

            ours = lambda: ops.linear_cross_entropy(hidden, weight, target, -1, 1.0)  # noqa: E731
            return dict(shape=[rows, d, vocab], work=6.0 * rows * d * vocab, kind="flops",
                        ours=ours, baseline=library)
        ours = lambda: ops.linear_cross_entropy(hidden, weight, target, -1, 1.0)  # noqa: E731
        base = lambda: F.cross_entropy((hidden @ weight.t()).float(), target, reduction="sum")  # noqa: E731
        return dict(shape=[rows, d, vocab], work=2.0 * rows * d * vocab, kind="flops", ours=ours,
                    baseline=base)
    return dict(shape=[rows, d], work=moved, kind="bytes", ours=ours, baseline=base)

def bench_rope(kind, args, timer):
    from ohara_b200.embeddings_pos.rotary import apply_rope, precompute_freqs_cis

    b, t, h, d = args.batch, args.seq, args.heads, args.head_dim
    q, k = bf(b, t, h, d), bf(b, t, args.kv_heads or h, d)
    cos, sin = (x.cuda() for x in precompute_freqs_cis(d, t, 10000.0))

    def eager():  # the reference's expression: fp32, interleaved pairs
        out = []
        for x in (q, k):
            xf = x.float().reshape(*x.shape[:-1], d // 2, 2)
            x0, x1 = xf.unbind(-1)
            c, s = cos[None, :, None, :], sin[None, :, None, :]
            out.append(torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), -1).flatten(-2).to(x.dtype))
        return out

    moved = 2.0 * (q.numel() + k.numel()) * 2
    return dict(shape=[b, t, h, d], work=moved, kind="bytes",
                ours=lambda: apply_rope(q, k, (cos, sin)), baseline=eager)


def bench_adamw(kind, args, timer):
    from ohara_b200.optimizer import FusedAdamW

    n = args.m * args.n
    p1 = torch.nn.Parameter(torch.randn(args.m, args.n, device="cuda"))
    p2 = torch.nn.Parameter(p1.detach().clone())
    p1.grad, p2.grad = torch.randn_like(p1), torch.randn_like(p2)
    ours_opt = FusedAdamW([p1], lr=1e-3, weight_decay=0.01)
    base_opt = torch.optim.AdamW([p2], lr=1e-3, weight_decay=0.01, foreach=True)
    return dict(shape=[args.m, args.n], work=7.0 * n * 4, kind="bytes", ours=ours_opt.step,
                baseline=base_opt.step)


def bench_newton_schulz(kind, args, timer):
    from ohara_b200.optimizer import POLAR_EXPRESS_COEFFICIENTS, _polar_express

    batch, r, c = args.batch, args.m, args.n
    g = torch.randn(batch, r, c, device="cuda")

    def library():  # the reference's iteration on batched cuBLAS
        x = g.bfloat16()
        x = x / (x.float().norm(dim=(-2, -1), keepdim=True).to(x.dtype) * 1.01 + 1e-6)
        for ca, cb, cc in POLAR_EXPRESS_COEFFICIENTS[:5]:
            if r > c:
                a = x.mT @ x
                x = ca * x + x @ (cb * a + cc * (a @ a))
            else:
                a = x @ x.mT
                x = ca * x + (cb * a + cc * (a @ a)) @ x
        return x

    side, long = min(r, c), max(r, c)
    flops = 5 * batch * (2.0 * side * side * long * 2 + 2.0 * side * side * side)
    return dict(shape=[batch, r, c], work=flops, kind="flops", ours=lambda: _polar_express(g, 5),
                baseline=library)


def _moe_inputs(args):
    tokens, dim, experts, k = args.m, args.n, args.experts, args.topk
    x = bf(tokens, dim)
    router = torch.randn(experts, dim, device="cuda") * dim ** -0.5
    return tokens, dim, experts, k, x, router


def bench_router(kind, args, timer):
    from ohara_b200.ops import moe

    tokens, dim, experts, k, x, router = _moe_inputs(args)
    bias = torch.zeros(experts, device="cuda")

    def ours():
        logits = moe.router_logits(x, router)
        return moe.route(logits, bias, k, "softmax", False, True)

    def library():  # the reference's routing: fp32 linear, top-(k+1), gather, softmax
        logits = F.linear(x.float(), router)
        top = torch.topk(logits + bias, k + 1, dim=-1)
        chosen = logits.gather(-1, top.indices[:, :k])
        return top.indices[:, :k], torch.softmax(chosen, -1), top.values[:, -1]

    return dict(shape=[tokens, dim, experts, k], work=2.0 * tokens * dim * experts, kind="flops",
                ours=ours, baseline=library)


def bench_permute_combine(kind, args, timer):
    from ohara_b200.ops import moe

    tokens, dim, experts, k, x, _ = _moe_inputs(args)
    indices = torch.stack([torch.randperm(experts, device="cuda")[:k] for _ in range(64)])
    indices = indices.repeat(tokens // 64, 1).int()
    weights = torch.rand(tokens, k, device="cuda")
    counts = torch.bincount(indices.reshape(-1), minlength=experts).int()

    def ours():
        dest_row, row_pair, _, _ = moe.dispatch_plan(indices, counts)
        padded = moe.permute_rows(x, dest_row, row_pair, k)
        return moe.combine_rows(padded, weights, dest_row, row_pair)

    def library():  # the reference's dispatch: stable argsort, gather, weighted index_add_
        flat = indices.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        rows = order // k
        torch.bincount(flat, minlength=experts).cumsum(0)
        gathered = x[rows]
        out = torch.zeros_like(x)
        return out.index_add_(0, rows, gathered * weights.reshape(-1)[order][:, None].to(x.dtype))

    return dict(shape=[tokens, dim, experts, k], work=4.0 * tokens * k * dim * 2, kind="bytes",
                ours=ours, baseline=library)


def bench_grouped_gemm(kind, args, timer):
    from ohara_b200.ops import grouped, moe

    tokens, dim, experts, k, x, _ = _moe_inputs(args)
    hidden = args.k
    weight = bf(experts, dim, hidden)
    indices = torch.randint(0, experts, (tokens, k), device="cuda").int()
    counts = torch.bincount(indices.reshape(-1), minlength=experts).int()
    dest_row, row_pair, tile_expert, k_offsets = moe.dispatch_plan(indices, counts)
    padded = moe.permute_rows(x, dest_row, row_pair, k)
    order = torch.argsort(indices.reshape(-1).long(), stable=True)
    sorted_x = x[order // k].contiguous()
    offsets = counts.cumsum(0).int()
    ours = lambda: grouped.grouped_linear(padded, weight, tile_expert, k_offsets)  # noqa: E731
    library = (lambda: torch._grouped_mm(sorted_x, weight, offs=offsets)) if hasattr(torch, "_grouped_mm") else ours
    return dict(shape=[tokens * k, dim, hidden, experts], work=2.0 * tokens * k * dim * hidden,
                kind="flops", ours=ours, baseline=library)


def bench_quantile(kind, args, timer):
    from ohara_b200.ops import moe

    tokens, _, experts, k, _, _ = _moe_inputs(args)
    logits = torch.randn(tokens, experts, device="cuda")
    alpha = torch.randn(tokens, device="cuda")
    beta = torch.zeros(experts, device="cuda")
    share = max(1, tokens * k // experts)
    ours = lambda: moe.accumulate_quantile(logits, alpha, beta, share)  # noqa: E731
    library = lambda: torch.topk((logits - alpha[:, None]).t(), share, dim=-1).values[:, -1]  # noqa: E731
    return dict(shape=[tokens, experts, share], work=1.0 * tokens * experts * 4, kind="bytes",
                ours=ours, baseline=library)


def bench_decode_attention(kind, args, timer):
    from ohara_b200.modules.kv_cache import KVCache
    from ohara_b200.ops import decode

    b, h, d, length = args.batch, args.heads, args.head_dim, args.seq
    hk = args.kv_heads or h
    cache = KVCache((b, length, hk, d), length, 0, device="cuda", dtype=torch.bfloat16)
    cache.key.normal_(), cache.value.normal_()
    cache.set_length(length, b)
    q = bf(b, 1, h, d)
    mask = torch.ones(1, length, dtype=torch.bool, device="cuda")

    def library():  # the reference's decode step: expand KV heads, SDPA with an explicit mask
        kk = cache.key.repeat_interleave(h // hk, dim=2).transpose(1, 2)
        vv = cache.value.repeat_interleave(h // hk, dim=2).transpose(1, 2)
        return F.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, attn_mask=mask)

    moved = 2.0 * b * length * hk * d * 2
    return dict(shape=[b, length, h, hk, d], work=moved, kind="bytes",
                ours=lambda: decode.decode_attention(q, cache, length - 1), baseline=library)


def bench_sampler(kind, args, timer):
    from ohara_b200.ops import decode

    rows, vocab = args.batch, args.n
    logits = torch.randn(rows, vocab, device="cuda").bfloat16()
    generator = torch.Generator(device="cuda").manual_seed(0)

    def library():  # the reference's sampler: top-k threshold, softmax, sorted top-p, multinomial
        last = logits.float()
        kth = last.topk(50, dim=-1).values[:, -1:]
        probs = torch.softmax(last.masked_fill(last < kth, float("-inf")), dim=-1)
        ordered, order = torch.sort(probs, dim=-1, descending=True)
        before = torch.cumsum(ordered, dim=-1) - ordered
        ordered = ordered.masked_fill(before > 0.9, 0.0)
        ordered = ordered / ordered.sum(dim=-1, keepdim=True)
        pick = torch.multinomial(ordered, num_samples=1, generator=generator)
        return torch.gather(order, -1, pick)

    ours = lambda: decode.sample(logits, temperature=1.0, top_k=50, top_p=0.9)  # noqa: E731
    return dict(shape=[rows, vocab], work=1.0 * rows * vocab * 2, kind="bytes", ours=ours,
                baseline=library)


def bench_pscan(kind, args, timer):
    """Linear-recurrence scan, forward + backward, against the whole-tensor doubling scan."""
    from ohara_b200.modules.pscan import PScan, pscan

    batch, length, channels = args.batch, args.seq, args.n
    a = torch.rand(batch, length, channels, device="cuda").mul_(0.2).add_(0.8).requires_grad_()
    x = torch.randn(batch, length, channels, device="cuda", requires_grad=True)
    grad = torch.randn(batch, length, channels, device="cuda")

    def run(fn):
        a.grad = x.grad = None
        fn(a, x).backward(grad)

    # forward reads a, x and writes h; backward reads dh, a, h and writes da, dx
    return dict(shape=[batch, length, channels], work=8.0 * batch * length * channels * 4,
                kind="bytes", ours=lambda: run(pscan), baseline=lambda: run(PScan.apply))


OPS = {
    "gemm_nt": bench_gemm, "gemm_nn": bench_gemm, "gemm_tn": bench_gemm,
    "attn_fwd": bench_attention, "attn_bwd": bench_attention,
    "rmsnorm": bench_bandwidth, "swiglu": bench_bandwidth, "linear_ce": bench_bandwidth,
    "linear_ce_train": bench_bandwidth,
    "rope": bench_rope, "adamw": bench_adamw, "newton_schulz": bench_newton_schulz,
    "router": bench_router, "permute_combine": bench_permute_combine,
    "grouped_gemm": bench_grouped_gemm, "quantile": bench_quantile,
    "decode_attention": bench_decode_attention, "sampler": bench_sampler,
    "pscan": bench_pscan,
}
DEFAULTS = {
    "gemm_nt": dict(m=65536, n=768, k=768), "gemm_nn": dict(m=65536, n=768, k=2048),
    "gemm_tn": dict(m=768, n=2048, k=65536), "rmsnorm": dict(m=65536, n=768),
    "swiglu": dict(m=65536, n=2048), "linear_ce": dict(m=8192, n=768, k=50304),
    "linear_ce_train": dict(m=8192, n=768, k=50304),
    "adamw": dict(m=50304, n=768), "newton_schulz": dict(m=768, n=768, batch=48),
    "router": dict(m=32768, n=1024), "permute_combine": dict(m=32768, n=1024),
    "grouped_gemm": dict(m=32768, n=1024, k=512), "quantile": dict(m=32768, n=1024),
    "decode_attention": dict(batch=64, seq=768), "sampler": dict(batch=64, n=50304),
    "pscan": dict(batch=4, seq=1024, n=24576),
}


def main() -> None:
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--op", choices=["all", *OPS], default="all")
    p.add_argument("--ops", default=None, help="comma-separated subset of operations (one process)")
    p.add_argument("--m", type=int, default=None)
    p.add_argument("--n", type=int, default=None)
    p.add_argument("--k", type=int, default=None)
    p.add_argument("--batch", type=int, default=None)
    p.add_argument("--seq", type=int, default=None)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--heads", type=int, default=6)
    p.add_argument("--kv-heads", type=int, default=0)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--no-baseline", action="store_true")
    args = p.parse_args()
    flop_peak, byte_peak = peaks()
    timer = Timer(args.iters, args.warmup)
    selected = list(OPS) if args.op == "all" else [args.op]
    if args.ops:
        selected = [name for name in args.ops.split(",") if name]
        unknown = [name for name in selected if name not in OPS]
        if unknown:
            p.error("unknown operations: " + ", ".join(unknown))
    for name in selected:
        local = argparse.Namespace(**vars(args))
        for key, value in {"batch": 32, "seq": 2048, **DEFAULTS.get(name, {})}.items():
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
