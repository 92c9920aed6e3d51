"""The CPU configuration of the benchmark set: a tiny Llama trained for 20 AdamW steps in fp32 on
one process (4 layers, width 256, 4 heads of 64, SwiGLU width 768, vocabulary 8192, tied
embeddings, sequence 256, batch 8; i.i.d. uniform tokens from seed 0; AdamW lr 3e-4, betas
(0.9, 0.95), weight decay 0.1).

    python examples/bench_cpu_tiny_llama.py                    # this package
    python examples/bench_cpu_tiny_llama.py --impl reference   # the reference package, if installed

Prints one JSON line: first and last loss, median step time after three warm-up steps, tokens per
second. Both arms run the same loop through the package's public API (``Llama``, ``Config``,
``build_adamw``); with the same seed they start from the same weights and see the same tokens, so
the losses must agree to rounding and only the step time may differ.
"""

from __future__ import annotations

import argparse
import importlib
import json
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--threads", type=int, default=8)
    args = parser.parse_args()

    import torch

    if args.impl == "reference":
        installed = ROOT / "baseline" / "_ref"
        if not (installed / "ohara").is_dir():
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
            return
        sys.path.insert(0, str(installed))
        package = "ohara"
    else:
        sys.path.insert(0, str(ROOT))
        package = "ohara_b200"
    library = importlib.import_module(package)
    optimizers = importlib.import_module(package + ".optimizer")

    torch.set_num_threads(args.threads)
    torch.manual_seed(0)
    model = library.Llama(library.Config(
        vocab_size=8192, hidden_size=256, intermediate_size=768, num_attention_heads=4,
        num_hidden_layers=4, max_sequence_length=256, weight_tying=True, dropout=0.0,
        rope_theta=10000))
    optimizer = optimizers.build_adamw(model, learning_rate=3e-4, weight_decay=0.1,
                                       betas=(0.9, 0.95))
    tokens_per_step = 8 * 256
    generator = torch.Generator().manual_seed(0)
    seconds, losses = [], []
    for _ in range(args.steps):
        tokens = torch.randint(0, 8192, (8, 257), generator=generator)
        started = time.perf_counter()
        logits = model(tokens[:, :-1])
        loss = torch.nn.functional.cross_entropy(
            logits.reshape(-1, logits.size(-1)).float(), tokens[:, 1:].reshape(-1))
        optimizer.zero_grad(set_to_none=True)
        loss.backward()
        optimizer.step()
        seconds.append(time.perf_counter() - started)
        losses.append(loss.item())
    median = statistics.median(seconds[3:] if len(seconds) > 3 else seconds)
    print(json.dumps({
        "impl": args.impl, "metric": "train tokens/sec", "value": tokens_per_step / median,
        "unit": "tokens/s", "device": "cpu", "dtype": "fp32", "threads": args.threads,
        "steps": args.steps, "warmup": min(3, max(0, len(seconds) - 1)),
        "ms_per_step": 1e3 * median, "first_loss": losses[0], "last_loss": losses[-1],
        "data": "synthetic", "config": {
            "model": "tiny llama (4L d256 4hx64 ffn768 V8192 tied)", "global_batch": 8,
            "seq_len": 256, "parallelism": "single process"}}))


if __name__ == "__main__":
    main()
