"""Dense vs mixture-of-experts training throughput at matched FLOPs per token.

    python examples/bench_moe.py --device-batch-size 8

Routing adds work that is not matmul (top-k, permutation, ragged expert GEMMs, combine), so at equal
FLOPs per token an MoE shows lower MFU than the dense model it replaces; what it buys is parameters
at constant compute. The MoE row shrinks each expert to ``intermediate_size // experts_per_tok`` so
the two rows differ in parameters, not in compute. Steps are timed on the device with CUDA events
(median over ``--steps``); MFU is against ``--peak-flops`` or, by default, the measured sustained
bf16 matmul rate of this machine when a ``MEASURED_PEAKS.json`` is present.
Flags follow the reference entry point (examples/bench_moe.py:30-46); ``--per-expert`` switches
from the grouped expert path to the per-expert module loop.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

import torch

from ohara_b200.models.llama import Config, Llama
from ohara_b200.modules.moe import apply_qb_update, expert_load, maximal_violation
from ohara_b200.optimizer import build_adamw
from ohara_b200.trainer import measured_peak_flops


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Compare dense and MoE throughput")
    p.add_argument("--hidden-size", type=int, default=768)
    p.add_argument("--intermediate-size", type=int, default=2048)
    p.add_argument("--num-layers", type=int, default=12)
    p.add_argument("--num-heads", type=int, default=6)
    p.add_argument("--vocab-size", type=int, default=50304)
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--device-batch-size", type=int, default=8)
    p.add_argument("--num-experts", type=int, default=8)
    p.add_argument("--experts-per-tok", type=int, default=2)
    p.add_argument("--moe-layer-interval", type=int, default=1)
    p.add_argument("--per-expert", action="store_true")
    p.add_argument("--steps", type=int, default=12)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--compile", action="store_true", help="accepted and ignored")
    p.add_argument("--peak-flops", type=float, default=None)
    return p.parse_args()


def build(args, *, moe: bool) -> Llama:
    width = args.intermediate_size // args.experts_per_tok if moe else args.intermediate_size
    return Llama(Config(
        vocab_size=args.vocab_size, hidden_size=args.hidden_size, intermediate_size=width,
        max_sequence_length=args.seq_len, num_hidden_layers=args.num_layers,
        num_attention_heads=args.num_heads, dropout=0.0, weight_tying=False, init_style="nanochat",
        moe_num_experts=args.num_experts if moe else 0, moe_experts_per_tok=args.experts_per_tok,
        moe_layer_interval=args.moe_layer_interval, moe_grouped=moe and not args.per_expert,
    ))


def benchmark(model: Llama, args, peak: float, *, moe: bool) -> dict[str, float]:
    device = torch.device("cuda")
    model = model.to(device)
    optimizer = build_adamw(model, learning_rate=1e-4, weight_decay=0.0)
    shape = (args.device_batch_size, args.seq_len)
    tokens = shape[0] * shape[1]
    # Fresh batches every step so no step reads inputs the previous one left in L2.
    batches = [(torch.randint(0, args.vocab_size, shape, device=device),
                torch.randint(0, args.vocab_size, shape, device=device)) for _ in range(4)]
    torch.cuda.reset_peak_memory_stats()
    times = []
    for step in range(args.warmup + args.steps):
        x, y = batches[step % len(batches)]
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
            loss = model(x, targets=y)
        loss.backward()
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        if moe:
            apply_qb_update(model)
        end.record()
        end.synchronize()
        if step >= args.warmup:
            times.append(begin.elapsed_time(end) / 1e3)
    median = sorted(times)[len(times) // 2]
    flops = model.estimate_flops(args.seq_len)
    row = {"step_s": median, "tokens_per_s": tokens / median,
           "mfu": 100.0 * flops * tokens / median / peak, "flops_per_token": flops,
           "params": sum(p.numel() for p in model.parameters()),
           "active": model.active_matmul_parameters(),
           "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9}
    if moe:
        per_layer = expert_load(model, reset=False)
        if per_layer is not None:
            row["maxvio"] = float(maximal_violation(per_layer).mean())
    del optimizer, model
    torch.cuda.empty_cache()
    return row


def main() -> None:
    args = parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark needs a CUDA device")
    peak = args.peak_flops or measured_peak_flops() or 2.25e15
    print(f"{args.num_layers}L hidden={args.hidden_size} seq={args.seq_len} "
          f"device_batch={args.device_batch_size} peak={peak / 1e12:.0f} TFLOP/s")
    print(f"MoE: {args.num_experts} experts, top-{args.experts_per_tok}, every "
          f"{args.moe_layer_interval} layer(s), expert width "
          f"{args.intermediate_size // args.experts_per_tok}, "
          f"{'per-expert loop' if args.per_expert else 'grouped'}\n")
    rows = {name: benchmark(build(args, moe=flag), args, peak, moe=flag)
            for name, flag in (("dense", False), ("moe", True))}
    header = f"{'':6} {'step':>9} {'tok/s':>11} {'MFU':>8} {'params':>12} {'active':>12} {'mem':>8}"
    print(header + "\n" + "-" * len(header))
    for name, r in rows.items():
        print(f"{name:6} {r['step_s']:8.3f}s {r['tokens_per_s']:11,.0f} {r['mfu']:7.1f}% "
              f"{r['params'] / 1e6:11.1f}M {r['active'] / 1e6:11.1f}M {r['peak_mem_gb']:7.1f}G")
    dense, moe = rows["dense"], rows["moe"]
    print(f"\nFLOPs/token: dense {dense['flops_per_token']:,.0f} vs moe {moe['flops_per_token']:,.0f} "
          f"({moe['flops_per_token'] / dense['flops_per_token']:.3f}x)")
    print(f"MoE has {moe['params'] / dense['params']:.2f}x the parameters, costs "
          f"{moe['step_s'] / dense['step_s']:.2f}x the time per step, "
          f"reaches {moe['mfu'] / dense['mfu']:.2f}x the dense MFU")
    if "maxvio" in moe:
        print(f"router MaxVio after {args.steps + args.warmup} steps: {moe['maxvio']:.3f} (0 = balanced)")


if __name__ == "__main__":
    main()
