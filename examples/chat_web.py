"""Browser chat UI for a finetuned checkpoint.

    python examples/chat_web.py --checkpoint ./ckpt/sft.pt      # then open http://localhost:8080

The server binds to localhost by default; reach a remote machine with an ssh port forward
(``ssh -N -L 8080:localhost:8080 user@host``) rather than ``--host 0.0.0.0`` where possible.
Flags follow the reference entry point (examples/chat_web.py:22-58).
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

import torch

from ohara_b200.chat_engine import ChatEngine, SamplingConfig
from ohara_b200.webui import serve


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Chat with a finetuned model in a browser")
    p.add_argument("--checkpoint", default="./ckpt/sft.pt")
    p.add_argument("--tokenizer-dir", default=None,
                   help="tokenizer saved beside the checkpoint (default: <checkpoint stem>/)")
    p.add_argument("--tokenizer", default="EleutherAI/gpt-neo-125m",
                   help="fallback when no tokenizer directory sits beside the checkpoint")
    p.add_argument("--moe-experts-per-tok", type=int, default=2)
    p.add_argument("--moe-gate-fn", choices=("softmax", "sigmoid"), default="softmax")
    p.add_argument("--moe-no-normalize-weights", action="store_true")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--device", default=None)
    p.add_argument("--dtype", default=None, choices=("float32", "bfloat16", "float16"),
                   help="default: bfloat16 on cuda, float32 on cpu")
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top-p", type=float, default=0.95)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--max-new-tokens", type=int, default=512)
    return p.parse_args()


def main() -> None:
    args = parse_args()
    engine = ChatEngine.from_checkpoint(
        args.checkpoint, tokenizer_dir=args.tokenizer_dir, tokenizer_name=args.tokenizer,
        device=args.device, dtype=getattr(torch, args.dtype) if args.dtype else None,
        moe_experts_per_tok=args.moe_experts_per_tok, moe_gate_fn=args.moe_gate_fn,
        moe_normalize_weights=not args.moe_no_normalize_weights,
    )
    info = engine.metadata(args.checkpoint)
    print(f"loaded {args.checkpoint}: {info['parameters'] / 1e6:.1f}M params, {info['layers']} layers, "
          f"ctx {info['context_length']}, on {info['device']} in {info['dtype']}")
    sampling = SamplingConfig(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                              max_new_tokens=min(args.max_new_tokens, info["context_length"]))
    serve(engine, host=args.host, port=args.port, checkpoint_path=args.checkpoint, sampling=sampling)


if __name__ == "__main__":
    main()
