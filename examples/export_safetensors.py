"""Turn a training checkpoint into publishable weights: ``model.safetensors`` + ``config.json``.

    python examples/export_safetensors.py --checkpoint ckpt/moe_d12.pt --out export/moe-base

A training ``.pt`` is a pickle with optimizer and RNG state and wrapper-prefixed keys: right for
resuming, wrong for publishing (it runs code on load, is several times the size of the weights,
and hides the architecture in tensor shapes). The config sidecar matters for mixture-of-experts
models in particular, because top-k, the gate function and weight normalisation leave no trace in
any shape. Flags follow the reference entry point (examples/export_safetensors.py:37-58).
"""

from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

import torch

from ohara_b200.chat_engine import config_from_state_dict, strip_wrapper_prefixes

# Rebuilt from the config at construction, or running statistics: not worth publishing.
DERIVED_BUFFERS = ("freq_cos", "freq_sin", "qb_beta_sum", "qb_beta_count", "expert_counts")


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Export a checkpoint to safetensors")
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--out", required=True, help="output directory")
    p.add_argument("--moe-experts-per-tok", type=int, default=2)
    p.add_argument("--moe-gate-fn", choices=("softmax", "sigmoid"), default="softmax")
    p.add_argument("--moe-no-normalize-weights", action="store_true")
    p.add_argument("--keep-derived-buffers", action="store_true",
                   help="also export rotary tables and router statistics")
    return p.parse_args()


def export(checkpoint_path: Path, out_dir: Path, *, moe_experts_per_tok: int = 2,
           moe_gate_fn: str = "softmax", moe_normalize_weights: bool = True,
           keep_derived_buffers: bool = False) -> dict[str, object]:
    from safetensors.torch import save_file

    if not checkpoint_path.exists():
        raise FileNotFoundError(f"checkpoint not found: {checkpoint_path}")
    checkpoint = torch.load(checkpoint_path, map_location="cpu", weights_only=False)
    state = {strip_wrapper_prefixes(k): v for k, v in checkpoint.get("model", checkpoint).items()}
    config = config_from_state_dict(state, moe_experts_per_tok=moe_experts_per_tok,
                                    moe_gate_fn=moe_gate_fn,
                                    moe_normalize_weights=moe_normalize_weights)
    # safetensors refuses aliased storage (tied embeddings, views), hence the clone.
    tensors = {
        key: value.detach().cpu().contiguous().clone()
        for key, value in state.items()
        if isinstance(value, torch.Tensor)
        and (keep_derived_buffers or not key.endswith(DERIVED_BUFFERS))
    }
    if not tensors:
        raise RuntimeError("no tensors found in checkpoint")
    out_dir.mkdir(parents=True, exist_ok=True)
    weights = out_dir / "model.safetensors"
    save_file(tensors, weights, metadata={"format": "pt", "source": checkpoint_path.name})
    payload = {"architecture": "ohara_b200.models.llama.Llama", "iteration": checkpoint.get("idx"),
               **asdict(config)}
    (out_dir / "config.json").write_text(json.dumps(payload, indent=2) + "\n", encoding="utf-8")
    return {"tensors": len(tensors), "parameters": sum(t.numel() for t in tensors.values()),
            "bytes": weights.stat().st_size, "config": payload}


def main() -> None:
    args = parse_args()
    result = export(Path(args.checkpoint), Path(args.out),
                    moe_experts_per_tok=args.moe_experts_per_tok, moe_gate_fn=args.moe_gate_fn,
                    moe_normalize_weights=not args.moe_no_normalize_weights,
                    keep_derived_buffers=args.keep_derived_buffers)
    config = result["config"]
    kind = (f"moe={config['moe_num_experts']}x top-{config['moe_experts_per_tok']}"
            if config["moe_num_experts"] else "dense")
    print(f"exported {args.checkpoint} -> {args.out}/model.safetensors")
    print(f"  {result['tensors']} tensors, {result['parameters']:,} params, "
          f"{result['bytes'] / 1e9:.2f} GB")
    print(f"  {config['num_hidden_layers']}L hidden={config['hidden_size']} "
          f"vocab={config['vocab_size']} {kind}")


if __name__ == "__main__":
    main()
