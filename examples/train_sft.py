"""Supervised finetuning: turn a pretrained Llama checkpoint into a chat model.

    python examples/train_sft.py --pretrained-checkpoint ./ckpt/base.pt

The architecture is recovered from the checkpoint's tensor shapes, the vocabulary grows by the chat
special tokens if pretraining did not reserve them, conversations are packed best-fit with
assistant-only loss masks, and a short warm-down pass runs at a fraction of the pretraining rates
with zero weight decay. The tokenizer and an ``ohara_chat.json`` metadata file are written beside
the checkpoint so the serving path can be started from that directory alone.
Flag surface follows the reference entry point (examples/train_sft.py:53-150); ``--conversations``
(a local JSONL of ``{"messages": [...]}`` rows) is added for machines without dataset access.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

import torch
from torch.utils.data import DataLoader

from ohara_b200 import Llama, OharaEngine, Trainer
from ohara_b200.chat import (
    ASSISTANT_END,
    CHAT_SPECIAL_TOKENS,
    load_chat_tokenizer,
    resize_token_embeddings,
    special_token_ids,
)
from ohara_b200.chat_engine import config_from_state_dict, strip_wrapper_prefixes
from ohara_b200.modules.moe import apply_qb_update
from ohara_b200.optimizer import build_adamw, build_muon_adamw
from ohara_b200.runtime import EngineConfig, ParallelConfig, PrecisionConfig, PrecisionMode
from ohara_b200.scaling import (
    CosineWeightDecayScheduler,
    MuonMomentumScheduler,
    WarmupStableDecayScheduler,
)
from ohara_b200.sft import ConversationDataset, build_mixture
from ohara_b200.tokenizer import get_token_bytes
from ohara_b200.tracking import BACKENDS as TRACKING_BACKENDS
from ohara_b200.tracking import create_logger

# Buffers that are rebuilt from the config or only track statistics; never a mismatch.
_DERIVED_BUFFERS = ("freq_cos", "freq_sin", "qb_beta_sum", "qb_beta_count", "expert_counts")


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Supervised finetune a pretrained Llama")
    p.add_argument("--pretrained-checkpoint", default="./ckpt/base.pt")
    p.add_argument("--checkpoint-path", default="./ckpt/sft.pt")
    p.add_argument("--tokenizer", default="EleutherAI/gpt-neo-125m")
    p.add_argument("--tokenizer-local-files-only", action="store_true")
    p.add_argument("--token-bytes-cache", default=None)
    # Three properties of an MoE base that no tensor shape records.
    p.add_argument("--moe-experts-per-tok", type=int, default=2)
    p.add_argument("--moe-gate-fn", choices=("softmax", "sigmoid"), default="softmax")
    p.add_argument("--moe-no-normalize-weights", action="store_true")

    p.add_argument("--conversations", default=None,
                   help="local JSONL with one {'messages': [...]} object per line; replaces the "
                        "downloaded SmolTalk / MMLU / GSM8K mixture (last 5%% is validation)")
    p.add_argument("--smoltalk-limit", type=int, default=None)
    p.add_argument("--mmlu-epochs", type=int, default=1)
    p.add_argument("--mmlu-limit", type=int, default=None)
    p.add_argument("--gsm8k-epochs", type=int, default=1)
    p.add_argument("--gsm8k-limit", type=int, default=None)
    p.add_argument("--val-smoltalk-limit", type=int, default=2_000)
    p.add_argument("--cache-dir", default=None)

    p.add_argument("--seq-len", type=int, default=None,
                   help="context length (default: the pretrained checkpoint's)")
    p.add_argument("--batch-size", type=int, default=8)
    p.add_argument("--grad-accum-steps", type=int, default=4)
    p.add_argument("--max-iters", type=int, default=800)
    p.add_argument("--eval-every", type=int, default=100)
    p.add_argument("--eval-batches", type=int, default=20)
    p.add_argument("--save-every", type=int, default=200)

    p.add_argument("--optimizer", choices=("muon", "adamw"), default="muon")
    p.add_argument("--matrix-learning-rate", type=float, default=0.02)
    p.add_argument("--embedding-learning-rate", type=float, default=0.3)
    p.add_argument("--unembedding-learning-rate", type=float, default=0.004)
    p.add_argument("--scalar-learning-rate", type=float, default=0.5)
    p.add_argument("--learning-rate", type=float, default=5e-5)
    p.add_argument("--init-lr-frac", type=float, default=0.8,
                   help="start at this fraction of the pretraining learning rates")
    p.add_argument("--warmup-iters", type=int, default=0)
    p.add_argument("--warmdown-ratio", type=float, default=0.5)
    p.add_argument("--final-lr-fraction", type=float, default=0.0)
    p.add_argument("--weight-decay", type=float, default=0.0)
    p.add_argument("--grad-clip-norm", type=float, default=1.0)

    p.add_argument("--logger", choices=TRACKING_BACKENDS, default="auto")
    p.add_argument("--project", default="ohara-sft")
    p.add_argument("--run-name", default=None)  # "--run" would collide with torchrun's --run-path
    p.add_argument("--precision", choices=[m.value for m in PrecisionMode],
                   default=PrecisionMode.BF16_MIXED.value)
    p.add_argument("--num-workers", type=int, default=0)
    p.add_argument("--buffer-size", type=int, default=100)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--tp", type=int, default=int(os.environ.get("OHARA_TP", "1")))
    p.add_argument("--evaluate-bpb", action="store_true")
    p.add_argument("--result-json", default=None)
    return p.parse_args()


def load_pretrained(path: Path, vocab_size: int, seq_len: int | None, **moe_hints):
    """Rebuild the base model from ``path`` and widen its vocabulary to ``vocab_size`` if needed.
    Returns ``(model, config, vocabulary size before widening)``."""
    if not path.exists():
        raise FileNotFoundError(f"pretrained checkpoint not found: {path}")
    checkpoint = torch.load(path, map_location="cpu", weights_only=False)
    state = {strip_wrapper_prefixes(k): v for k, v in checkpoint.get("model", checkpoint).items()}
    config = config_from_state_dict(state, **moe_hints)
    base_vocab = config.vocab_size
    if seq_len is not None:
        if seq_len > config.max_sequence_length:
            raise ValueError(f"--seq-len {seq_len} exceeds the pretrained context window "
                             f"of {config.max_sequence_length}")
        config.max_sequence_length = seq_len
    model = Llama(config)
    state = {k: v for k, v in state.items() if not k.startswith(("freq_cos", "freq_sin"))}
    missing, unexpected = model.load_state_dict(state, strict=False)
    missing = [k for k in missing if not k.endswith(_DERIVED_BUFFERS)]
    unexpected = [k for k in unexpected if not k.endswith(_DERIVED_BUFFERS)]
    if missing or unexpected:
        raise RuntimeError("checkpoint does not match the reconstructed model: "
                           f"missing={missing} unexpected={unexpected}")
    # A base trained with a padded vocabulary is wider than the tokenizer; keep the spare rows.
    if base_vocab < vocab_size:
        resize_token_embeddings(model, vocab_size)
    return model, config, base_vocab


def load_conversations(args):
    if args.conversations is not None:
        rows = [json.loads(line)
                for line in Path(args.conversations).read_text(encoding="utf-8").splitlines()
                if line.strip()]
        if not rows or not all(isinstance(row, dict) and "messages" in row for row in rows):
            raise ValueError(f"{args.conversations}: every line must be an object with a "
                             f"'messages' list")
        random.Random(args.seed).shuffle(rows)
        held_out = max(1, len(rows) // 20)
        return rows[held_out:], rows[:held_out]
    train = build_mixture(split="train", smoltalk_limit=args.smoltalk_limit,
                          mmlu_epochs=args.mmlu_epochs, mmlu_limit=args.mmlu_limit,
                          gsm8k_epochs=args.gsm8k_epochs, gsm8k_limit=args.gsm8k_limit,
                          cache_dir=args.cache_dir, seed=args.seed)
    val = build_mixture(split="val", smoltalk_limit=args.val_smoltalk_limit,
                        cache_dir=args.cache_dir, seed=args.seed)
    return train, val


def run() -> None:
    args = parse_args()
    if min(args.batch_size, args.grad_accum_steps, args.max_iters) < 1:
        raise ValueError("batch-size, grad-accum-steps and max-iters must be at least 1")
    if not 0 < args.init_lr_frac <= 1:
        raise ValueError("init-lr-frac must be in (0, 1]")
    if args.weight_decay < 0 or args.grad_clip_norm < 0:
        raise ValueError("weight-decay and grad-clip-norm cannot be negative")
    random.seed(args.seed)
    torch.manual_seed(args.seed)

    engine = OharaEngine(EngineConfig(precision=PrecisionConfig(mode=PrecisionMode(args.precision)),
                                      parallel=ParallelConfig(tp=args.tp)))
    engine.launch()
    tokenizer = load_chat_tokenizer(hf_name=args.tokenizer, prefer_hf=True,
                                    local_files_only=args.tokenizer_local_files_only)
    vocab = len(tokenizer)
    raw_model, config, base_vocab = load_pretrained(
        Path(args.pretrained_checkpoint), vocab, args.seq_len,
        moe_experts_per_tok=args.moe_experts_per_tok, moe_gate_fn=args.moe_gate_fn,
        moe_normalize_weights=not args.moe_no_normalize_weights)
    seq_len = config.max_sequence_length
    model = engine.prepare(raw_model)
    parameters = sum(p.numel() for p in raw_model.parameters())
    if engine.is_global_zero:
        print(f"loaded {args.pretrained_checkpoint}: depth={config.num_hidden_layers} "
              f"hidden={config.hidden_size} heads={config.num_attention_heads} ctx={seq_len} "
              f"params={parameters:,}")
        if base_vocab < vocab:
            print(f"grew vocabulary {base_vocab:,} -> {vocab:,} for "
                  f"{len(CHAT_SPECIAL_TOKENS)} chat special tokens")

    frac = args.init_lr_frac
    if args.optimizer == "muon":
        if args.tp != 1:
            raise ValueError("the hybrid Muon optimizer currently requires --tp 1")
        optimizer = build_muon_adamw(
            model, matrix_learning_rate=args.matrix_learning_rate * frac,
            embedding_learning_rate=args.embedding_learning_rate * frac,
            unembedding_learning_rate=args.unembedding_learning_rate * frac,
            scalar_learning_rate=args.scalar_learning_rate * frac, weight_decay=args.weight_decay)
        base_lr = args.matrix_learning_rate * frac
    else:
        optimizer = build_adamw(model, learning_rate=args.learning_rate * frac,
                                weight_decay=args.weight_decay)
        base_lr = args.learning_rate * frac
    optimizer = engine.prepare_optimizers(optimizer)[0]

    tracker = None
    if engine.is_global_zero:  # one run per job, not one per rank
        tracker = create_logger(args.logger, project=args.project, run_name=args.run_name, config={
            **vars(args), "vocab_size": vocab, "parameters": parameters,
            "depth": config.num_hidden_layers, "world_size": engine.data_parallel_world_size})
        engine.loggers = [tracker]

    train_rows, val_rows = load_conversations(args)
    if engine.is_global_zero:
        print(f"mixture: {len(train_rows):,} train / {len(val_rows):,} val conversations")
    shared = dict(tokenizer=tokenizer, max_length=seq_len, buffer_size=args.buffer_size,
                  data_rank=engine.data_parallel_rank,
                  data_world_size=engine.data_parallel_world_size)
    loader = dict(batch_size=args.batch_size, num_workers=args.num_workers,
                  pin_memory=engine.device.type == "cuda")
    train_dl, val_dl = engine.prepare_dataloaders(
        DataLoader(ConversationDataset(train_rows, shuffle=True, seed=args.seed, **shared), **loader),
        DataLoader(ConversationDataset(val_rows, shuffle=False, seed=args.seed + 1, **shared), **loader),
    )

    get_lr = WarmupStableDecayScheduler(learning_rate=base_lr, max_iters=args.max_iters,
                                        warmup_iters=args.warmup_iters,
                                        warmdown_ratio=args.warmdown_ratio,
                                        final_lr_fraction=args.final_lr_fraction)
    get_hparams = None
    if args.optimizer == "muon":
        momentum = MuonMomentumScheduler(max_iters=args.max_iters,
                                         warmdown_ratio=args.warmdown_ratio, warmup_iters=0)
        decay = CosineWeightDecayScheduler(weight_decay=args.weight_decay, max_iters=args.max_iters)

        def get_hparams(iteration: int) -> dict[str, float]:
            return {"momentum": momentum(iteration), "weight_decay": decay(iteration)}

    token_bytes = (get_token_bytes(tokenizer, device=engine.device, cache_path=args.token_bytes_cache)
                   if args.evaluate_bpb else None)
    trainer = Trainer(
        engine=engine, model=model, optimizer=optimizer, train_dataloader=train_dl,
        val_dataloader=val_dl, get_lr=get_lr, get_optimizer_hparams=get_hparams,
        micro_batch=args.grad_accum_steps, max_iters=args.max_iters, eval_iters=args.eval_every,
        save_ckpt_iters=args.save_every, ignore_index=-1, print_every=10,
        eval_val_batches=args.eval_batches, grad_clip_norm=args.grad_clip_norm or None,
        checkpoint_path=args.checkpoint_path, token_bytes=token_bytes,
        apply_router_balancing=apply_qb_update if config.moe_num_experts > 0 else None,
    )

    initial = trainer.evaluate(trainer.val_dataloader, args.eval_batches)
    if engine.is_global_zero:
        print(f"before SFT: val_loss={initial['loss']:.4f} val_ppl={initial['ppl']:.2f} "
              f"val_acc={initial['accuracy']:.4f}")
    started = time.perf_counter()
    trainer.train()
    wall_time = time.perf_counter() - started
    final = trainer.evaluate(trainer.val_dataloader, args.eval_batches)

    if engine.is_global_zero:
        print(f"after SFT: val_loss={final['loss']:.4f} val_ppl={final['ppl']:.2f} "
              f"val_acc={final['accuracy']:.4f} time={wall_time / 60:.1f}m")
        bundle = Path(args.checkpoint_path).with_suffix("")
        bundle.mkdir(parents=True, exist_ok=True)
        tokenizer.save_pretrained(bundle)
        metadata = {
            "vocab_size": vocab, "hidden_size": config.hidden_size,
            "intermediate_size": config.intermediate_size,
            "num_hidden_layers": config.num_hidden_layers,
            "num_attention_heads": config.num_attention_heads,
            "num_key_value_heads": config.num_key_value_heads,
            "max_sequence_length": config.max_sequence_length,
            "weight_tying": config.weight_tying, "tokenizer": args.tokenizer,
            "assistant_end_id": special_token_ids(tokenizer)[ASSISTANT_END],
            "initial_val_loss": initial["loss"], "val_loss": final["loss"],
            "val_accuracy": final["accuracy"], "max_iters": args.max_iters,
            "train_time_sec": wall_time,
        }
        text = json.dumps(metadata, indent=2) + "\n"
        (bundle / "ohara_chat.json").write_text(text, encoding="utf-8")
        print(f"saved chat tokenizer and metadata to {bundle}")
        if args.result_json is not None:
            Path(args.result_json).parent.mkdir(parents=True, exist_ok=True)
            Path(args.result_json).write_text(text, encoding="utf-8")
    if tracker is not None:
        tracker.finish()
    engine.close()


if __name__ == "__main__":
    run()
