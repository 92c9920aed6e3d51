"""Pretrain a Llama with ``OharaEngine`` + ``Trainer``.

Single GPU:   python examples/train_llama_engine.py --dataset ./corpus --optimizer muon ...
Multi GPU:    torchrun --nproc-per-node 8 examples/train_llama_engine.py --strategy fsdp ...

Flag surface follows the reference entry point (examples/train_llama_engine.py:39-187) and adds
``--strategy`` (``fsdp`` = sharded optimizer with fused NVLink collectives), ``--cp`` / ``--ep``
and ``--synthetic`` (uniform random tokens, for benchmarking without a dataset or a tokenizer).
Token bins (``{split}.bin`` beside the corpus, see pretokenize_corpus.py) are preferred over
tokenising inside the loop.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

import torch
from torch.utils.data import DataLoader, IterableDataset

from ohara_b200 import Config, CosineScheduler, Llama, OharaEngine, Trainer
from ohara_b200.modules.moe import apply_qb_update
from ohara_b200.optimizer import build_adamh, build_adamw, build_muon_adamw, build_muonh_adamh
from ohara_b200.runtime import (
    EngineConfig,
    FaultToleranceConfig,
    ParallelConfig,
    PipelinePlan,
    PrecisionConfig,
    PrecisionMode,
    StrategyType,
    TensorParallelPlan,
)
from ohara_b200.scaling import (
    CosineWeightDecayScheduler,
    MuonMomentumScheduler,
    WarmupStableDecayScheduler,
)
from ohara_b200.tracking import BACKENDS as TRACKING_BACKENDS
from ohara_b200.tracking import create_logger


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Train a Llama on streamed or pre-tokenised text")
    data = p.add_argument_group("data")
    data.add_argument("--dataset", default="roneneldan/TinyStories")
    data.add_argument("--dataset-config", default=None)
    data.add_argument("--tokenizer", default="EleutherAI/gpt-neo-125m")
    data.add_argument("--tokenizer-local-files-only", action="store_true")
    data.add_argument("--token-bytes-cache", default=None)
    data.add_argument("--chat-tokens", action="store_true",
                      help="reserve the chat special tokens now so SFT need not grow the vocabulary")
    data.add_argument("--text-column", default="text")
    data.add_argument("--train-split", default="train")
    data.add_argument("--validation-split", default="validation")
    data.add_argument("--no-token-bins", action="store_true",
                      help="ignore {split}.bin files and tokenise text inline")
    data.add_argument("--pad-vocab-to", type=int, default=1,
                      help="round the model vocabulary up to a multiple of this")
    data.add_argument("--num-workers", type=int, default=0)
    data.add_argument("--synthetic", action="store_true",
                      help="uniform random tokens (needs --synthetic-vocab); no dataset, no tokenizer")
    data.add_argument("--synthetic-vocab", type=int, default=50304)

    shape = p.add_argument_group("model")
    shape.add_argument("--seq-len", type=int, default=256)
    shape.add_argument("--hidden-size", type=int, default=256)
    shape.add_argument("--intermediate-size", type=int, default=1_024)
    shape.add_argument("--num-layers", type=int, default=6)
    shape.add_argument("--num-heads", type=int, default=8)
    shape.add_argument("--num-kv-heads", type=int, default=0)
    shape.add_argument("--dropout", type=float, default=0.0)
    shape.add_argument("--init-style", choices=("standard", "nanochat"), default="standard")
    shape.add_argument("--weight-tying", action=argparse.BooleanOptionalAction, default=True)
    shape.add_argument("--moe-num-experts", type=int, default=0)
    shape.add_argument("--moe-experts-per-tok", type=int, default=2)
    shape.add_argument("--moe-layer-interval", type=int, default=1)
    shape.add_argument("--moe-gate-fn", choices=("softmax", "sigmoid"), default="softmax")
    shape.add_argument("--moe-grouped", action="store_true")
    shape.add_argument("--moe-num-shared-experts", type=int, default=0)
    shape.add_argument("--moe-no-normalize-weights", action="store_true")
    shape.add_argument("--moe-no-quantile-balancing", action="store_true")
    shape.add_argument("--moe-aux-loss-coef", type=float, default=0.0)
    shape.add_argument("--moe-capacity-factor", type=float, default=None)

    opt = p.add_argument_group("optimisation")
    opt.add_argument("--batch-size", type=int, default=8)
    opt.add_argument("--grad-accum-steps", type=int, default=4)
    opt.add_argument("--max-iters", type=int, default=10_000)
    opt.add_argument("--optimizer", choices=("adamw", "muon", "adamh", "muonh"), default="adamw")
    opt.add_argument("--learning-rate", type=float, default=5e-4)
    opt.add_argument("--matrix-learning-rate", type=float, default=0.02)
    opt.add_argument("--embedding-learning-rate", type=float, default=0.3)
    opt.add_argument("--unembedding-learning-rate", type=float, default=0.008)
    opt.add_argument("--scalar-learning-rate", type=float, default=0.5)
    opt.add_argument("--hypersphere-learning-rate", type=float, default=None)
    opt.add_argument("--min-lr", type=float, default=5e-5)
    opt.add_argument("--weight-decay", type=float, default=0.1)
    opt.add_argument("--muon-momentum-warmup-iters", type=int, default=400)
    opt.add_argument("--grad-clip-norm", type=float, default=1.0)
    opt.add_argument("--warmup-iters", type=int, default=100)
    opt.add_argument("--lr-schedule", choices=("cosine", "wsd"), default="cosine")
    opt.add_argument("--warmdown-ratio", type=float, default=0.65)
    opt.add_argument("--final-lr-fraction", type=float, default=0.05)

    run = p.add_argument_group("run")
    run.add_argument("--eval-every", type=int, default=200)
    run.add_argument("--eval-batches", type=int, default=20)
    run.add_argument("--save-every", type=int, default=1_000)
    run.add_argument("--checkpoint-path", default="./ckpt/model.pt")
    run.add_argument("--resume", action="store_true")
    run.add_argument("--evaluate-bpb", action="store_true")
    run.add_argument("--result-json", default=None)
    run.add_argument("--scaling-depth", type=int, default=None)
    run.add_argument("--flops-budget", type=float, default=None)
    run.add_argument("--logger", choices=TRACKING_BACKENDS, default="auto")
    run.add_argument("--project", default="ohara")
    run.add_argument("--run-name", default=None)
    run.add_argument("--compile", action="store_true",
                     help="accepted for command-line compatibility; the hot ops are hand-written "
                          "kernels, so there is nothing for a tracing compiler to do")
    run.add_argument("--seed", type=int, default=42)
    run.add_argument("--tp", type=int, default=int(os.environ.get("OHARA_TP", "1")))
    run.add_argument("--cp", type=int, default=1)
    run.add_argument("--ep", type=int, default=1)
    run.add_argument("--pp", type=int, default=1,
                     help="pipeline stages (GPipe order through the trainer; needs --no-weight-tying)")
    run.add_argument("--pp-micro-batch-size", type=int, default=1,
                     help="sequences per pipeline micro-batch")
    run.add_argument("--dp-replicate", type=int, default=1,
                     help="with --strategy fsdp: replica groups of a hybrid-sharded run")
    run.add_argument("--sequence-parallel", action="store_true")
    run.add_argument("--strategy", choices=[s.value for s in StrategyType], default="auto")
    run.add_argument("--heartbeat-interval", type=float, default=0.0,
                     help="seconds between heartbeats over the rendezvous store (0 = off); a rank "
                          "whose heartbeat stops is reported before the next step is launched")
    run.add_argument("--heartbeat-timeout", type=float, default=30.0)
    run.add_argument("--context-parallel-mode", choices=["ring", "ulysses"], default="ring",
                     help="with --cp > 1: key/value exchange under the flash kernels (ring) or "
                          "all-to-all between sequence shards and head shards (ulysses)")
    run.add_argument("--shard-parameters", action="store_true",
                     help="with --strategy fsdp: shard the parameters per transformer block "
                          "(gathered just before a block runs) instead of the optimizer state "
                          "alone")
    run.add_argument("--shard-parameters-layout", choices=["auto", "even", "matrix"], default="auto",
                     help="even: equal ranges (AdamW); matrix: whole matrices at one owner (Muon; "
                          "AdamH / MuonH are not supported with sharded parameters); auto picks by "
                          "--optimizer")
    run.add_argument("--activation-checkpointing", action="store_true",
                     help="recompute every block in the backward pass instead of keeping its "
                          "activations (less memory, about a third more compute)")
    run.add_argument("--profile-sections", action="store_true",
                     help="time the phases of every step on the device (CUDA events, max over "
                          "ranks) and print the totals at the end; OHARA_NVTX=1 adds NVTX ranges")
    run.add_argument("--step-timeout", type=float, default=0.0,
                     help="abort (exit code 75) when one training step takes longer than this "
                          "many seconds (0 = off), so that an elastic launcher can restart the job")
    run.add_argument("--precision", choices=[m.value for m in PrecisionMode],
                     default=PrecisionMode.BF16_MIXED.value)
    return p.parse_args()


def validate(args: argparse.Namespace) -> None:
    checks = [
        (args.hidden_size % args.num_heads == 0, "hidden-size must be divisible by num-heads"),
        (args.grad_accum_steps >= 1, "grad-accum-steps must be at least 1"),
        (args.batch_size >= 1 and args.max_iters >= 1, "batch-size and max-iters must be at least 1"),
        (args.eval_every >= 0 and args.eval_batches >= 1 and args.save_every >= 0,
         "invalid evaluation or checkpoint interval"),
        (args.num_workers >= 0, "num-workers cannot be negative"),
        (0.0 <= args.dropout < 1.0, "dropout must be in [0, 1)"),
        (args.pad_vocab_to >= 1, "pad-vocab-to must be at least 1"),
    ]
    for ok, message in checks:
        if not ok:
            raise ValueError(message)


class SyntheticTokens(IterableDataset):
    """Endless i.i.d. uniform token rows; the stream differs per data-parallel rank."""

    def __init__(self, vocab: int, seq_len: int, seed: int) -> None:
        self.vocab, self.seq_len, self.seed = vocab, seq_len, seed

    def __iter__(self):
        gen = torch.Generator().manual_seed(self.seed)
        while True:
            row = torch.randint(0, self.vocab, (self.seq_len + 1,), generator=gen)
            yield row[:-1], row[1:]


def build_optimizer(args, model):
    """Returns ``(optimizer, learning rate the schedule is expressed in)``."""
    if args.optimizer == "muon":
        return build_muon_adamw(
            model, matrix_learning_rate=args.matrix_learning_rate,
            embedding_learning_rate=args.embedding_learning_rate,
            unembedding_learning_rate=args.unembedding_learning_rate,
            scalar_learning_rate=args.scalar_learning_rate, weight_decay=args.weight_decay,
        ), args.matrix_learning_rate
    if args.optimizer in ("adamh", "muonh"):
        # On the sphere the rate is a relative step; sqrt(lr * wd) carries an additive recipe over.
        additive = args.matrix_learning_rate if args.optimizer == "muonh" else args.learning_rate
        rate = args.hypersphere_learning_rate
        if rate is None:
            rate = math.sqrt(additive * args.weight_decay)
            if rate <= 0:
                raise ValueError("cannot derive a hyperspherical learning rate from --weight-decay 0; "
                                 "pass --hypersphere-learning-rate explicitly")
        builder = build_muonh_adamh if args.optimizer == "muonh" else build_adamh
        adam_rate = args.embedding_learning_rate if args.optimizer == "muonh" else args.learning_rate
        return builder(model, learning_rate=rate, adam_learning_rate=adam_rate), rate
    return build_adamw(model, learning_rate=args.learning_rate,
                       weight_decay=args.weight_decay), args.learning_rate


def build_datasets(args, engine, tokenizer):
    rank, world = engine.data_parallel_rank, engine.data_parallel_world_size
    if args.synthetic:
        return (SyntheticTokens(args.synthetic_vocab, args.seq_len, args.seed + 1000 * rank),
                SyntheticTokens(args.synthetic_vocab, args.seq_len, args.seed + 7 + 1000 * rank))
    from ohara_b200.dataset import StreamingTextDataset
    from ohara_b200.tokenbin import TokenBinDataset

    corpus = Path(args.dataset)
    train_bin = corpus / f"{args.train_split}.bin"
    val_bin = corpus / f"{args.validation_split}.bin"
    if not args.no_token_bins and train_bin.exists() and val_bin.exists():
        common = dict(max_length=args.seq_len, tokenizer=tokenizer, data_rank=rank,
                      data_world_size=world, seed=args.seed)
        train, val = (TokenBinDataset(train_bin, shuffle=True, **common),
                      TokenBinDataset(val_bin, shuffle=False, **common))
        if engine.is_global_zero:
            print(f"token bins: train {train.metadata['tokens']:,} tokens, "
                  f"val {val.metadata['tokens']:,} tokens")
        return train, val
    common = dict(dataset_name=args.dataset, name=args.dataset_config, tokenizer=tokenizer,
                  max_length=args.seq_len, text_column=args.text_column, data_rank=rank,
                  data_world_size=world, seed=args.seed)
    return (StreamingTextDataset(**common, split=args.train_split, shuffle=True),
            StreamingTextDataset(**common, split=args.validation_split, shuffle=False))


def build_schedules(args, base_lr: float):
    if args.lr_schedule == "wsd":
        lr = WarmupStableDecayScheduler(learning_rate=base_lr, max_iters=args.max_iters,
                                        warmup_iters=args.warmup_iters,
                                        warmdown_ratio=args.warmdown_ratio,
                                        final_lr_fraction=args.final_lr_fraction)
    else:
        lr = CosineScheduler(learning_rate=base_lr, min_lr=args.min_lr,
                             warmup_iters=args.warmup_iters, max_iters=args.max_iters)
    hparams = None
    if args.optimizer == "muon":
        momentum = MuonMomentumScheduler(max_iters=args.max_iters,
                                         warmdown_ratio=args.warmdown_ratio,
                                         warmup_iters=args.muon_momentum_warmup_iters)
        decay = CosineWeightDecayScheduler(weight_decay=args.weight_decay, max_iters=args.max_iters)

        def hparams(iteration: int) -> dict[str, float]:
            return {"momentum": momentum(iteration), "weight_decay": decay(iteration)}

    return lr, hparams


def resume(args, engine, model, optimizer, trainer, train_ds) -> int:
    checkpoint = engine.load(args.checkpoint_path, {"model": model, "optimizer": optimizer})
    start = int(checkpoint["idx"])
    saved_accum = int(checkpoint.get("gradient_accumulation_steps", args.grad_accum_steps))
    if saved_accum != args.grad_accum_steps:
        raise ValueError("checkpoint gradient accumulation does not match --grad-accum-steps")
    consumed = int(checkpoint.get("train_batches_consumed", start * args.grad_accum_steps))
    if consumed > 0 and args.num_workers != 0:
        raise ValueError("exact --resume currently requires --num-workers 0")
    if hasattr(train_ds, "start_block"):
        train_ds.start_block = consumed * args.batch_size
    trainer.train_batches_consumed = consumed
    if "torch_rng_state" in checkpoint:
        torch.set_rng_state(checkpoint["torch_rng_state"].cpu())
    if torch.cuda.is_available() and "cuda_rng_state_all" in checkpoint:
        torch.cuda.set_rng_state_all(checkpoint["cuda_rng_state_all"])
    if engine.is_global_zero:
        print(f"resumed checkpoint={args.checkpoint_path} at iter={start}; "
              f"skipping {consumed * args.batch_size:,} previously consumed blocks")
    return start


def write_result(args, engine, model, base_lr, initial, final, wall_time) -> None:
    counts = model.num_scaling_params()
    flops_per_token = model.estimate_flops(args.seq_len)
    batch_tokens = (args.batch_size * args.seq_len * args.grad_accum_steps
                    * engine.data_parallel_world_size)
    tokens = args.max_iters * batch_tokens
    result = {
        "flops_budget": args.flops_budget if args.flops_budget is not None else flops_per_token * tokens,
        "depth": args.scaling_depth if args.scaling_depth is not None else args.num_layers,
        "hidden_size": args.hidden_size, "intermediate_size": args.intermediate_size,
        "num_heads": args.num_heads, "sequence_length": args.seq_len,
        "params_token_embeddings": counts["token_embeddings"], "params_lm_head": counts["lm_head"],
        "params_transformer": counts["transformer_matrices"],
        "params_norms_and_scalars": counts["norms_and_scalars"], "params_total": counts["total"],
        "params_effective": counts["effective"], "flops_per_token": flops_per_token,
        "total_batch_size": batch_tokens, "num_iterations": args.max_iters,
        "tokens_trained": tokens, "actual_training_flops": flops_per_token * tokens,
        "tokens_per_effective_param": tokens / counts["effective"], "optimizer": args.optimizer,
        "optimizer_muon": float(args.optimizer == "muon"),
        "initialization_nanochat": float(args.init_style == "nanochat"),
        "learning_rate": base_lr, "matrix_learning_rate": args.matrix_learning_rate,
        "embedding_learning_rate": args.embedding_learning_rate,
        "unembedding_learning_rate": args.unembedding_learning_rate,
        "scalar_learning_rate": args.scalar_learning_rate, "weight_decay": args.weight_decay,
        "initial_val_loss": initial["loss"], "initial_val_bpb": initial.get("bpb", float("nan")),
        "val_loss": final["loss"], "val_bpb": final.get("bpb", float("nan")),
        "val_bits_per_token": final["bits_per_token"], "train_time_sec": wall_time,
    }
    path = Path(args.result_json)
    path.parent.mkdir(parents=True, exist_ok=True)
    temporary = path.with_name(f".{path.name}.tmp-{os.getpid()}")
    try:
        temporary.write_text(json.dumps(result, indent=2) + "\n", encoding="utf-8")
        os.replace(temporary, path)
    finally:
        temporary.unlink(missing_ok=True)


def run() -> None:
    args = parse_args()
    validate(args)
    torch.manual_seed(args.seed)

    engine = OharaEngine(EngineConfig(
        strategy=StrategyType(args.strategy),
        precision=PrecisionConfig(mode=PrecisionMode(args.precision)),
        parallel=ParallelConfig(tp=args.tp, cp=args.cp, ep=args.ep, pp=args.pp,
                                dp_replicate=args.dp_replicate),
        pipeline=(PipelinePlan(degree=args.pp, micro_batch_size=args.pp_micro_batch_size)
                  if args.pp > 1 else PipelinePlan()),
        tensor_parallel=TensorParallelPlan.llama_default(args.tp, args.sequence_parallel),
        activation_checkpointing=args.activation_checkpointing,
        shard_parameters=args.shard_parameters,
        shard_parameters_layout=(args.shard_parameters_layout if args.shard_parameters_layout != "auto"
                                 else ("even" if args.optimizer == "adamw" else "matrix")),
        context_parallel_mode=args.context_parallel_mode,
        fault_tolerance=FaultToleranceConfig(
            heartbeat_interval_s=args.heartbeat_interval, heartbeat_timeout_s=args.heartbeat_timeout,
            step_timeout_s=args.step_timeout, exit_on_step_timeout=args.step_timeout > 0),
    ))
    engine.launch()

    tokenizer = None
    if args.synthetic:
        tokenizer_vocab = args.synthetic_vocab
    else:
        from ohara_b200.chat import add_chat_tokens
        from ohara_b200.tokenizer import get_tokenizer

        tokenizer = get_tokenizer(hf_name=args.tokenizer, prefer_hf=True,
                                  local_files_only=args.tokenizer_local_files_only)
        if args.chat_tokens:
            add_chat_tokens(tokenizer)
        tokenizer_vocab = len(tokenizer)
    # Padding the vocabulary only adds rows that no target ever selects.
    vocab = -(-tokenizer_vocab // args.pad_vocab_to) * args.pad_vocab_to

    raw_model = Llama(Config(
        vocab_size=vocab, hidden_size=args.hidden_size, intermediate_size=args.intermediate_size,
        max_sequence_length=args.seq_len, num_hidden_layers=args.num_layers,
        num_attention_heads=args.num_heads, num_key_value_heads=args.num_kv_heads,
        dropout=args.dropout, multiple_of=4, weight_tying=args.weight_tying,
        init_style=args.init_style, moe_num_experts=args.moe_num_experts,
        moe_experts_per_tok=args.moe_experts_per_tok, moe_layer_interval=args.moe_layer_interval,
        moe_gate_fn=args.moe_gate_fn, moe_quantile_balancing=not args.moe_no_quantile_balancing,
        moe_grouped=args.moe_grouped, moe_num_shared_experts=args.moe_num_shared_experts,
        moe_normalize_weights=not args.moe_no_normalize_weights,
        moe_aux_loss_coef=args.moe_aux_loss_coef, moe_capacity_factor=args.moe_capacity_factor,
    ))
    model = engine.prepare(raw_model)
    optimizer, base_lr = build_optimizer(args, model)
    optimizer = engine.prepare_optimizers(optimizer)[0]

    tracker = None
    if engine.is_global_zero:
        tracker = create_logger(args.logger, project=args.project, run_name=args.run_name, config={
            **vars(args), "vocab_size": vocab,
            "parameters": sum(p.numel() for p in raw_model.parameters()),
            "world_size": engine.data_parallel_world_size,
        })
        engine.loggers = [tracker]

    train_ds, val_ds = build_datasets(args, engine, tokenizer)
    loader = dict(batch_size=args.batch_size, num_workers=args.num_workers,
                  pin_memory=engine.device.type == "cuda")
    train_dl, val_dl = engine.prepare_dataloaders(
        DataLoader(train_ds, **loader, generator=torch.Generator().manual_seed(args.seed)),
        DataLoader(val_ds, **loader, generator=torch.Generator().manual_seed(args.seed + 1)),
    )
    get_lr, get_hparams = build_schedules(args, base_lr)

    token_bytes = None
    if args.evaluate_bpb and tokenizer is not None:
        from ohara_b200.tokenizer import get_token_bytes

        token_bytes = get_token_bytes(tokenizer, device=engine.device, cache_path=args.token_bytes_cache)
        if token_bytes.numel() < vocab:  # padded ids carry zero bytes
            token_bytes = torch.nn.functional.pad(token_bytes, (0, vocab - token_bytes.numel()))

    balancing = args.moe_num_experts > 0 and not args.moe_no_quantile_balancing
    trainer = Trainer(
        engine=engine, model=model, optimizer=optimizer, train_dataloader=train_dl,
        val_dataloader=val_dl, get_lr=get_lr, get_optimizer_hparams=get_hparams,
        micro_batch=args.grad_accum_steps, max_iters=args.max_iters, eval_iters=args.eval_every,
        save_ckpt_iters=args.save_every, ignore_index=-1, print_every=1,
        eval_val_batches=args.eval_batches, eval_train_batches=0,
        grad_clip_norm=args.grad_clip_norm or None, timing_warmup_steps=10,
        checkpoint_path=args.checkpoint_path, token_bytes=token_bytes,
        apply_router_balancing=apply_qb_update if balancing else None,
        profile_sections=args.profile_sections,
    )
    start_iter = resume(args, engine, model, optimizer, trainer, train_ds) if args.resume else 0

    initial = trainer.evaluate(trainer.val_dataloader, args.eval_batches)
    if engine.is_global_zero:
        params = sum(p.numel() for p in raw_model.parameters())
        tokens_per_step = args.batch_size * args.seq_len * args.grad_accum_steps
        note = f" vocab={tokenizer_vocab:,}->{vocab:,}" if vocab != tokenizer_vocab else ""
        print(f"device={engine.device} precision={args.precision} strategy={type(engine.strategy).__name__} "
              f"params={params:,} tokens/step/rank={tokens_per_step:,} max_iters={args.max_iters:,}"
              f"{note} random_loss={math.log(tokenizer_vocab):.4f}")
        print(f"starting val_loss={initial['loss']:.4f} val_ppl={initial['ppl']:.2f} "
              f"val_bits/token={initial['bits_per_token']:.4f}")

    started = time.perf_counter()
    trainer.train(start_iter=start_iter)
    wall_time = time.perf_counter() - started
    sections = trainer.section_times()  # a collective: every rank takes part
    if sections and engine.is_global_zero:
        print("device time per phase (max over ranks): " + ", ".join(
            f"{name}={entry['ms'] / max(entry['calls'], 1):.2f} ms x {entry['calls']}"
            for name, entry in sections.items()))
    final = trainer.evaluate(trainer.val_dataloader, args.eval_batches)
    if engine.is_global_zero:
        line = (f"final val_loss={final['loss']:.4f} val_ppl={final['ppl']:.2f} "
                f"val_bits/token={final['bits_per_token']:.4f}")
        if "bpb" in final:
            line += f" val_bpb={final['bpb']:.4f}"
        print(line)
        if args.result_json is not None:
            write_result(args, engine, raw_model, base_lr, initial, final, wall_time)
    if tracker is not None:
        tracker.finish()
    engine.close()


if __name__ == "__main__":
    run()
