"""CORE in-context-learning evaluation of a checkpoint of this package or a Hugging Face model.

    python examples/core_eval.py --checkpoint ckpt/model.pt --chat-tokens
    python examples/core_eval.py --hf-model openai-community/gpt2 --max-per-task 100

Flags follow the reference entry point (examples/core_eval.py:19-77).
"""

from __future__ import annotations

import argparse
import json
import sys
from contextlib import nullcontext
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

import torch

from ohara_b200.chat import add_chat_tokens
from ohara_b200.chat_engine import config_from_state_dict, strip_wrapper_prefixes
from ohara_b200.core_eval import evaluate_core
from ohara_b200.models.llama import Llama
from ohara_b200.tokenizer import get_tokenizer
from ohara_b200.utils import auto_accelerator


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Run CORE-style evaluation")
    p.add_argument("--hf-model", default="openai-community/gpt2",
                   help="Hugging Face model id (ignored when --checkpoint is given)")
    p.add_argument("--checkpoint", default=None, help="a .pt written by the trainers")
    p.add_argument("--tokenizer", default="EleutherAI/gpt-neo-125m", help="tokenizer for --checkpoint")
    p.add_argument("--chat-tokens", action="store_true",
                   help="extend the tokenizer with the chat special tokens, as training did")
    p.add_argument("--moe-experts-per-tok", type=int, default=2)
    p.add_argument("--moe-gate-fn", choices=("softmax", "sigmoid"), default="softmax")
    p.add_argument("--moe-no-normalize-weights", action="store_true")
    p.add_argument("--label", default=None, help="name for the result row")
    p.add_argument("--output-json", default=None)
    p.add_argument("--max-per-task", type=int, default=100, help="-1 for all")
    p.add_argument("--eval-bundle-dir", default="./eval_bundle")
    p.add_argument("--dtype", default="auto", choices=["auto", "float32", "bfloat16"])
    return p.parse_args()


def load_checkpoint_model(args, device, dtype):
    checkpoint = torch.load(args.checkpoint, map_location="cpu", weights_only=False)
    state = {strip_wrapper_prefixes(k): v for k, v in checkpoint.get("model", checkpoint).items()}
    config = config_from_state_dict(state, moe_experts_per_tok=args.moe_experts_per_tok,
                                    moe_gate_fn=args.moe_gate_fn,
                                    moe_normalize_weights=not args.moe_no_normalize_weights)
    model = Llama(config)
    model.load_state_dict(state, strict=False)
    kind = (f"moe={config.moe_num_experts}x top-{config.moe_experts_per_tok}"
            if config.moe_num_experts else "dense")
    print(f"loaded {args.checkpoint}: {config.num_hidden_layers}L hidden={config.hidden_size} "
          f"vocab={config.vocab_size} {kind}")
    return model.to(device=device, dtype=dtype)


def main() -> None:
    args = parse_args()
    device = auto_accelerator()
    if args.dtype == "auto":
        dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    else:
        dtype = getattr(torch, args.dtype)

    if args.checkpoint:
        tokenizer = get_tokenizer(hf_name=args.tokenizer, prefer_hf=True)
        if args.chat_tokens:
            add_chat_tokens(tokenizer)
        model = load_checkpoint_model(args, device, dtype)
    else:
        from transformers import AutoModelForCausalLM

        tokenizer = get_tokenizer(hf_name=args.hf_model, prefer_hf=True)
        model = AutoModelForCausalLM.from_pretrained(args.hf_model, torch_dtype=dtype).to(device)
    model.eval()

    autocast = (torch.amp.autocast(device_type="cuda", dtype=dtype)
                if device.type == "cuda" and dtype != torch.float32 else nullcontext())
    with autocast:
        results = evaluate_core(model=model, tokenizer=tokenizer, device=device,
                                max_per_task=args.max_per_task,
                                eval_bundle_dir=args.eval_bundle_dir)
    label = args.label or args.checkpoint or args.hf_model
    print(json.dumps(results, indent=2))
    print(f"CORE  {label}: {results['core_metric']:.4f}")
    if args.output_json:
        Path(args.output_json).write_text(json.dumps({"label": label, **results}, indent=2) + "\n",
                                          encoding="utf-8")


if __name__ == "__main__":
    main()
