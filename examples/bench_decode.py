"""KV-cache decode throughput of the depth-12 Llama: prompt of 512 uniform-random tokens, 256 new
tokens, temperature 1.0, top-k 50, top-p 0.9, bf16, batch 1 / 16 / 64 on one GPU.

    python examples/bench_decode.py                     # this package (fused kernels + CUDA graph)
    python examples/bench_decode.py --no-graph          # same kernels, launched eagerly
    python examples/bench_decode.py --impl reference    # the reference package, if installed

The timed region is the whole generation (prefill + every decode step) between CUDA events after
``--warmup`` untimed generations; tokens/s counts generated tokens over all sequences. One JSON line
per batch size. The reference arm drives the reference's own model, KV cache and
``sample_next_token`` in the loop its chat engine uses (chat_engine.py:368-412), widened to a batch.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Decode throughput benchmark")
    p.add_argument("--impl", choices=("ours", "reference"), default="ours")
    p.add_argument("--batches", default="1,16,64")
    p.add_argument("--prompt-len", type=int, default=512)
    p.add_argument("--new-tokens", type=int, default=256)
    p.add_argument("--repeats", type=int, default=3)
    p.add_argument("--warmup", type=int, default=1)
    p.add_argument("--no-graph", action="store_true")
    p.add_argument("--int8-cache", action="store_true")
    p.add_argument("--tp", type=int, default=1,
                   help="tensor-parallel degree; launch with torchrun --nproc-per-node <tp>")
    return p.parse_args()


MODEL = dict(vocab_size=50304, hidden_size=768, intermediate_size=2048, num_hidden_layers=12,
             num_attention_heads=6, max_sequence_length=2048, dropout=0.0, weight_tying=False)
SAMPLING = dict(temperature=1.0, top_k=50, top_p=0.9)


def time_generations(torch, generate, repeats: int, warmup: int) -> float:
    for _ in range(warmup):
        generate()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(repeats):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        generate()
        end.record()
        end.synchronize()
        best = min(best, begin.elapsed_time(end) / 1e3)
    return best


def run_ours(args):
    sys.path.insert(0, str(ROOT))
    import torch

    from ohara_b200.chat_engine import ChatEngine, SamplingConfig
    from ohara_b200.models.llama import Config, Llama

    class Vocabulary:  # the engine only needs the special-token ids and the vocabulary size
        eos_token_id = bos_token_id = pad_token_id = 0

        def __len__(self):
            return MODEL["vocab_size"]

        def get_vocab(self):
            from ohara_b200.chat import CHAT_SPECIAL_TOKENS

            return {token: MODEL["vocab_size"] - 1 - i for i, token in enumerate(CHAT_SPECIAL_TOKENS)}

    torch.manual_seed(0)
    model = Llama(Config(**MODEL))
    device, rank0, heads_split = "cuda", True, True
    if args.tp > 1:
        # Attention heads and the feed-forward width are sharded over the ranks; the all-reduce
        # behind each row-parallel layer is the one-shot peer-memory kernel, replayed from the
        # same CUDA graph as the rest of the decode step.
        from ohara_b200.runtime import EngineConfig, OharaEngine, ParallelConfig, TensorParallelPlan

        # When the degree does not divide the head count (6 heads on 4 or 8 ranks) only the
        # feed-forward layers and the output head are sharded and attention is replicated.
        heads_split = MODEL["num_attention_heads"] % args.tp == 0
        plan = (TensorParallelPlan.llama_default(args.tp) if heads_split
                else TensorParallelPlan.mlp_and_head(args.tp))
        runtime = OharaEngine(EngineConfig(parallel=ParallelConfig(tp=args.tp),
                                           tensor_parallel=plan))
        runtime.launch()
        model = runtime.prepare_module(model.to(torch.bfloat16))
        device, rank0 = runtime.device, runtime.is_global_zero
    engine = ChatEngine(model, Vocabulary(), device=device, dtype=torch.bfloat16)
    config = SamplingConfig(max_new_tokens=args.new_tokens, **SAMPLING)
    for batch in (int(b) for b in args.batches.split(",")):
        prompt = torch.randint(0, MODEL["vocab_size"], (batch, args.prompt_len), device=device)
        seconds = time_generations(
            torch, lambda: engine.generate_batch(prompt, config, seed=1, cuda_graph=not args.no_graph),
            args.repeats, args.warmup)
        if rank0:
            plan_name = "none" if args.tp == 1 else ("heads+mlp" if heads_split else "mlp+head")
            report(args, "ours", batch, seconds,
                   {"cuda_graph": not args.no_graph, "tp": args.tp, "tp_plan": plan_name})


def run_reference(args):
    sys.path.insert(0, str(ROOT / "baseline" / "stubs"))
    sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
    if not (ROOT / "baseline" / "_ref" / "ohara").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/ohara is missing"}))
        return
    import torch

    from ohara.chat_engine import SamplingConfig, sample_next_token  # the reference package
    from ohara.models.llama import Config, Llama

    torch.manual_seed(0)
    model = Llama(Config(**MODEL)).to(device="cuda", dtype=torch.bfloat16).eval()
    config = SamplingConfig(max_new_tokens=args.new_tokens, **SAMPLING)

    @torch.inference_mode()
    def generate(prompt):
        cache = model.build_kv_cache(batch_size=prompt.size(0))
        generator = torch.Generator(device="cuda").manual_seed(1)
        step_input, position = prompt, 0
        for _ in range(args.new_tokens):
            logits = model(step_input, cache, position)
            position += step_input.size(1)
            step_input = sample_next_token(logits, config, generator)
        return step_input

    for batch in (int(b) for b in args.batches.split(",")):
        prompt = torch.randint(0, MODEL["vocab_size"], (batch, args.prompt_len), device="cuda")
        seconds = time_generations(torch, lambda: generate(prompt), args.repeats, args.warmup)
        report(args, "reference", batch, seconds, {})


def report(args, impl: str, batch: int, seconds: float, extra: dict) -> None:
    print(json.dumps({
        "impl": impl, "metric": "decode tokens/sec", "value": batch * args.new_tokens / seconds,
        "unit": "tokens/s", "batch": batch, "prompt_len": args.prompt_len,
        "new_tokens": args.new_tokens, "seconds": seconds,
        "ms_per_token": 1e3 * seconds / args.new_tokens, "dtype": "bf16", "data": "synthetic",
        "sampling": SAMPLING, **extra,
    }), flush=True)


if __name__ == "__main__":
    arguments = parse_args()
    run_reference(arguments) if arguments.impl == "reference" else run_ours(arguments)
