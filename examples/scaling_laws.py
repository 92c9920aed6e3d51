"""Plan, run and analyse nanochat-style iso-FLOP sweeps of Llama models.

    python examples/scaling_laws.py plan    --depths 10,12,14 --flops-budgets 1e18,2e18
    python examples/scaling_laws.py run     --dataset ./data/scaling_corpus --results-dir ./scaling_results
    python examples/scaling_laws.py analyze --results-file ./scaling_results/results.csv --output-svg fit.svg

``run`` launches train_llama_engine.py once per (budget, depth) cell, checks that what was trained
is what was planned, and appends one numeric row per cell to ``results.csv``. A manifest beside the
results pins everything that must stay fixed within one fit; a sweep that would re-read a small
staged corpus more than ``--max-corpus-epochs`` times is refused.
Sub-commands and flags follow the reference entry point (examples/scaling_laws.py:42-151).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
from collections.abc import Mapping
from pathlib import Path

PROJECT_ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(PROJECT_ROOT))  # run from a source checkout

from ohara_b200.scaling import (
    ScalingPlan,
    analyze_scaling_results,
    append_result_csv,
    load_result_csv,
    plan_scaling_run,
    write_scaling_svg,
)

TRAIN_SCRIPT = PROJECT_ROOT / "examples" / "train_llama_engine.py"
SCALING_RECIPE_VERSION = 3

# argparse destination -> plan_scaling_run keyword, for the arguments that shape a plan.
_PLAN_KEYWORDS = {
    "vocab_size": "vocab_size", "seq_len": "sequence_length",
    "device_batch_size": "device_batch_size", "nproc_per_node": "world_size",
    "total_batch_size": "total_batch_size", "aspect_ratio": "aspect_ratio", "head_dim": "head_dim",
    "ffn_multiplier": "ffn_multiplier", "ffn_multiple_of": "ffn_multiple_of",
    "reference_depth": "reference_depth", "reference_batch_size": "reference_batch_size",
    "reference_tokens_per_param": "reference_tokens_per_param", "batch_exponent": "batch_exponent",
    "base_learning_rate": "base_learning_rate",
    "base_embedding_learning_rate": "base_embedding_learning_rate",
    "base_unembedding_learning_rate": "base_unembedding_learning_rate",
    "base_scalar_learning_rate": "base_scalar_learning_rate",
    "base_weight_decay": "base_weight_decay",
}
# Result fields that must equal the plan for a cell to count.
_PLANNED_FIELDS = ("matrix_learning_rate", "embedding_learning_rate", "unembedding_learning_rate",
                   "scalar_learning_rate", "weight_decay", "flops_per_token")


def _positive_list(cast):
    def parse(text: str):
        values = [cast(item) for item in text.split(",") if item.strip()]
        if not values or any(v <= 0 for v in values):
            raise argparse.ArgumentTypeError("expected comma-separated positive numbers")
        return values
    return parse


def _add_plan_arguments(p: argparse.ArgumentParser) -> None:
    ints, floats = _positive_list(int), _positive_list(float)
    p.add_argument("--depths", type=ints, default=ints("10,12,14,16,18,20"))
    p.add_argument("--flops-budgets", type=floats, default=floats("1e18,2.15e18,4.64e18,1e19"))
    p.add_argument("--vocab-size", type=int, default=50_257)
    p.add_argument("--seq-len", type=int, default=2_048)
    p.add_argument("--device-batch-size", type=int, default=32)
    p.add_argument("--nproc-per-node", type=int, default=1)
    p.add_argument("--total-batch-size", type=int, default=None)
    p.add_argument("--aspect-ratio", type=int, default=64)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--ffn-multiplier", type=float, default=8 / 3)
    p.add_argument("--ffn-multiple-of", type=int, default=256)
    p.add_argument("--reference-depth", type=int, default=12)
    p.add_argument("--reference-batch-size", type=int, default=2**19)
    p.add_argument("--reference-tokens-per-param", type=float, default=12.0)
    p.add_argument("--batch-exponent", type=float, default=0.383)
    p.add_argument("--base-matrix-learning-rate", "--base-learning-rate", dest="base_learning_rate",
                   type=float, default=0.02)
    p.add_argument("--base-embedding-learning-rate", type=float, default=0.3)
    p.add_argument("--base-unembedding-learning-rate", type=float, default=0.008)
    p.add_argument("--base-scalar-learning-rate", type=float, default=0.5)
    p.add_argument("--base-weight-decay", type=float, default=0.28)


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="Plan, run and analyse iso-FLOP Llama sweeps")
    sub = parser.add_subparsers(dest="command", required=True)

    plan = sub.add_parser("plan", help="print run configurations without training")
    _add_plan_arguments(plan)
    plan.add_argument("--output-json", default=None)

    run = sub.add_parser("run", help="execute the fixed-FLOP sweep")
    _add_plan_arguments(run)
    run.add_argument("--dataset", default="./data/scaling_corpus")
    run.add_argument("--dataset-config", default=None)
    run.add_argument("--tokenizer", default="EleutherAI/gpt-neo-125m")
    run.add_argument("--tokenizer-local-files-only", action="store_true")
    run.add_argument("--text-column", default="text")
    run.add_argument("--train-split", default="train")
    run.add_argument("--validation-split", default="validation")
    run.add_argument("--optimizer", choices=("muon", "muonh"), default="muon",
                     help="muon: Muon+AdamW; muonh: hyperspherical MuonH+AdamH")
    run.add_argument("--hypersphere-learning-rate", type=float, default=None,
                     help="fixed relative step for muonh across the whole grid; omitted, each run "
                          "derives sqrt(matrix_lr * weight_decay)")
    run.add_argument("--eval-batches", type=int, default=20)
    run.add_argument("--warmup-steps", type=int, default=40, help="ceiling; see --warmup-fraction")
    run.add_argument("--warmup-fraction", type=float, default=0.1)
    run.add_argument("--muon-momentum-warmup-iters", type=int, default=400, help="ceiling")
    run.add_argument("--warmdown-ratio", type=float, default=0.65)
    run.add_argument("--final-lr-fraction", type=float, default=0.05)
    run.add_argument("--precision", choices=("fp32", "fp16_mixed", "bf16_mixed", "bf16_true"),
                     default="bf16_mixed")
    run.add_argument("--strategy", choices=("auto", "single", "ddp", "fsdp"), default="auto")
    run.add_argument("--num-workers", type=int, default=0)
    run.add_argument("--seed", type=int, default=42)
    run.add_argument("--results-dir", default="./scaling_results")
    run.add_argument("--dry-run", action="store_true")
    run.add_argument("--max-corpus-epochs", type=float, default=3.0)
    run.add_argument("--allow-repeated-epochs", action="store_true")

    analyze = sub.add_parser("analyze", help="fit iso-FLOP curves")
    analyze.add_argument("--results-file", default="./scaling_results/results.csv")
    analyze.add_argument("--metric", default="val_bpb")
    analyze.add_argument("--output-json", default=None)
    analyze.add_argument("--output-svg", default=None)
    return parser.parse_args(argv)


def build_plans(args) -> list[ScalingPlan]:
    keywords = {name: getattr(args, dest) for dest, name in _PLAN_KEYWORDS.items()}
    return [plan_scaling_run(depth, flops_budget=budget, **keywords)
            for budget in args.flops_budgets for depth in args.depths]


def print_plans(plans: list[ScalingPlan]) -> None:
    print("budget,depth,dim,params,effective_params,batch,accum,iters,tokens,actual_flops,"
          "matrix_lr,embedding_lr,unembedding_lr,scalar_lr,wd")
    for p in plans:
        cells = [f"{p.flops_budget:.6g}", p.depth, p.hidden_size, p.params_total, p.params_effective,
                 p.total_batch_size, p.grad_accum_steps, p.num_iterations, p.tokens_trained,
                 f"{p.actual_training_flops:.6g}", f"{p.matrix_learning_rate:.6g}",
                 f"{p.embedding_learning_rate:.6g}", f"{p.unembedding_learning_rate:.6g}",
                 f"{p.scalar_learning_rate:.6g}", f"{p.weight_decay:.6g}"]
        print(",".join(str(c) for c in cells))


def scaled_warmup_iters(ceiling: int, num_iterations: int, fraction: float) -> int:
    """A warm-up length that never dominates the short runs of a sweep: iteration counts on one
    iso-FLOP curve differ by more than 100x, so a fixed count would train the cells under
    different effective schedules."""
    return max(1, min(ceiling, round(fraction * num_iterations)))


def training_command(args, plan: ScalingPlan, result_json: Path) -> list[str]:
    launcher = [sys.executable]
    if args.nproc_per_node > 1:
        launcher += ["-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                     f"--nproc_per_node={args.nproc_per_node}"]
    options = {
        "dataset": args.dataset, "tokenizer": args.tokenizer, "text-column": args.text_column,
        "train-split": args.train_split, "validation-split": args.validation_split,
        "seq-len": plan.sequence_length, "batch-size": plan.device_batch_size,
        "grad-accum-steps": plan.grad_accum_steps, "max-iters": plan.num_iterations,
        "eval-every": plan.num_iterations, "eval-batches": args.eval_batches, "save-every": 0,
        "optimizer": args.optimizer, "matrix-learning-rate": plan.matrix_learning_rate,
        "embedding-learning-rate": plan.embedding_learning_rate,
        "unembedding-learning-rate": plan.unembedding_learning_rate,
        "scalar-learning-rate": plan.scalar_learning_rate, "weight-decay": plan.weight_decay,
        "warmup-iters": scaled_warmup_iters(args.warmup_steps, plan.num_iterations,
                                            args.warmup_fraction),
        "muon-momentum-warmup-iters": scaled_warmup_iters(
            args.muon_momentum_warmup_iters, plan.num_iterations, args.warmup_fraction),
        "hidden-size": plan.hidden_size, "intermediate-size": plan.intermediate_size,
        "num-layers": plan.depth, "num-heads": plan.num_heads, "init-style": "nanochat",
        "lr-schedule": "wsd", "warmdown-ratio": args.warmdown_ratio,
        "final-lr-fraction": args.final_lr_fraction, "grad-clip-norm": 0,
        "token-bytes-cache": Path(args.results_dir) / "token_bytes.pt",
        "precision": args.precision, "strategy": args.strategy, "num-workers": args.num_workers,
        "seed": args.seed, "tp": 1, "result-json": result_json, "scaling-depth": plan.depth,
        "flops-budget": plan.flops_budget,
    }
    if args.dataset_config is not None:
        options["dataset-config"] = args.dataset_config
    if args.optimizer == "muonh" and args.hypersphere_learning_rate is not None:
        options["hypersphere-learning-rate"] = args.hypersphere_learning_rate
    command = launcher + [str(TRAIN_SCRIPT)]
    for name, value in options.items():
        command += [f"--{name}", str(value)]
    command += ["--no-weight-tying", "--evaluate-bpb"]
    if args.tokenizer_local_files_only:
        command.append("--tokenizer-local-files-only")
    return command


def experiment_manifest(args) -> dict[str, object]:
    """Everything that must stay fixed within one fitted sweep."""
    fixed = {
        "recipe_version": SCALING_RECIPE_VERSION,
        "optimizer": "muon_adamw" if args.optimizer == "muon" else "muonh_adamh",
        "initialization": "nanochat", "sequence_length": args.seq_len,
        "world_size": args.nproc_per_node, "base_matrix_learning_rate": args.base_learning_rate,
        "warmup_steps_ceiling": args.warmup_steps,
        "muon_momentum_warmup_iters_ceiling": args.muon_momentum_warmup_iters,
    }
    same_name = (
        "hypersphere_learning_rate", "dataset", "dataset_config", "tokenizer",
        "tokenizer_local_files_only", "text_column", "train_split", "validation_split",
        "vocab_size", "device_batch_size", "total_batch_size", "aspect_ratio", "head_dim",
        "ffn_multiplier", "ffn_multiple_of", "reference_depth", "reference_batch_size",
        "reference_tokens_per_param", "batch_exponent", "base_embedding_learning_rate",
        "base_unembedding_learning_rate", "base_scalar_learning_rate", "base_weight_decay",
        "warmup_fraction", "warmdown_ratio", "final_lr_fraction", "eval_batches", "precision",
        "num_workers", "seed",
    )
    fixed.update({name: getattr(args, name) for name in same_name})
    return fixed


def prepare_results_manifest(args, results_dir: Path) -> None:
    path = results_dir / "experiment.json"
    expected = experiment_manifest(args)
    if path.exists():
        recorded = json.loads(path.read_text(encoding="utf-8"))
        if recorded != expected:
            differing = sorted(k for k in set(recorded) | set(expected)
                               if recorded.get(k) != expected.get(k))
            raise ValueError(f"{path} does not match this run ({', '.join(differing)}); "
                             "use a fresh --results-dir")
        return
    if (results_dir / "results.csv").exists():
        raise ValueError(f"{results_dir} has results but no experiment manifest; use a fresh "
                         "--results-dir so incompatible runs cannot be mixed")
    results_dir.mkdir(parents=True, exist_ok=True)
    temporary = path.with_name(f".{path.name}.tmp-{os.getpid()}")
    try:
        temporary.write_text(json.dumps(expected, indent=2) + "\n", encoding="utf-8")
        os.replace(temporary, path)
    finally:
        temporary.unlink(missing_ok=True)


def corpus_token_budget(dataset: str) -> int | None:
    """Token count recorded by prepare_scaling_data.py, or ``None`` when there is none (not a
    staged corpus, or staged without a tokenizer); the epoch check is then skipped."""
    stats = Path(dataset) / "stats.train.json"
    if not stats.exists():
        return None
    tokens = json.loads(stats.read_text(encoding="utf-8")).get("tokens")
    return None if tokens is None else int(tokens)


def check_corpus_epoch_budget(args, plans: list[ScalingPlan]) -> None:
    """The streaming dataset loops its source forever without warning, so a token horizon beyond
    the corpus size would silently measure memorisation."""
    corpus = corpus_token_budget(args.dataset)
    if corpus is None:
        return
    epochs = max(p.tokens_trained for p in plans) / corpus
    print(f"corpus tokens={corpus:,}; sweep max epochs over corpus={epochs:.2f}")
    if epochs > args.max_corpus_epochs and not args.allow_repeated_epochs:
        raise ValueError(
            f"sweep would repeat the staged corpus at {args.dataset!r} up to {epochs:.1f}x, above "
            f"--max-corpus-epochs={args.max_corpus_epochs}; stage more documents with "
            "prepare_scaling_data.py, shrink --depths/--flops-budgets, or pass "
            "--allow-repeated-epochs to proceed anyway")


def numeric_result_row(result: Mapping[str, object]) -> dict[str, object]:
    """The CSV loader turns every column into a float, so descriptive strings stay out of it (the
    manifest records them)."""
    return {k: v for k, v in result.items()
            if isinstance(v, (int, float)) and not isinstance(v, bool)}


def verify_result(args, plan: ScalingPlan, result: Mapping[str, object]) -> None:
    if int(result["params_effective"]) != plan.params_effective:
        raise RuntimeError("trained model does not match the planned parameter count")
    if int(result["total_batch_size"]) != plan.total_batch_size:
        raise RuntimeError("training result does not match planned total_batch_size")
    if result.get("optimizer") not in (None, args.optimizer):
        raise RuntimeError(f"training result used optimizer {result.get('optimizer')!r}, not the "
                           f"planned {args.optimizer!r}")
    if result.get("optimizer_muon") != float(args.optimizer == "muon"):
        raise RuntimeError("training result did not use the planned optimizer recipe")
    if result.get("initialization_nanochat") != 1.0:
        raise RuntimeError("training result did not use the planned nanochat initialization")
    for name in _PLANNED_FIELDS:
        if not math.isclose(float(result[name]), float(getattr(plan, name))):
            raise RuntimeError(f"training result does not match planned {name}")


def run_sweep(args, plans: list[ScalingPlan]) -> None:
    results_dir = Path(args.results_dir)
    results_file = results_dir / "results.csv"
    if not args.dry_run:
        from ohara_b200.tokenizer import get_tokenizer

        size = len(get_tokenizer(hf_name=args.tokenizer, prefer_hf=True,
                                 local_files_only=args.tokenizer_local_files_only))
        if size != args.vocab_size:
            raise ValueError(f"--vocab-size={args.vocab_size} does not match tokenizer size {size}; "
                             "fix the plan before launching GPU runs")
        check_corpus_epoch_budget(args, plans)
        prepare_results_manifest(args, results_dir)
    finished: set[tuple[float, int]] = set()
    if results_file.exists():
        rows = load_result_csv(results_file)
        if any(r.get("optimizer_muon", 0.0) != float(args.optimizer == "muon") for r in rows):
            raise ValueError(f"{results_file} was produced with a different optimizer recipe than "
                             f"--optimizer={args.optimizer}; use a fresh --results-dir")
        finished = {(float(r["flops_budget"]), int(r["depth"])) for r in rows}

    for plan in plans:
        cell = (float(plan.flops_budget), plan.depth)
        if cell in finished:
            print(f"skip budget={plan.flops_budget:.6g} depth={plan.depth}: already complete")
            continue
        tag = f"flops_{plan.flops_budget:.6g}_d{plan.depth}".replace("+", "")
        result_json = results_dir / f"{tag}.json"
        command = training_command(args, plan, result_json)
        print("run:", " ".join(command))
        if args.dry_run:
            continue
        subprocess.run(command, cwd=PROJECT_ROOT, check=True)
        result = json.loads(result_json.read_text(encoding="utf-8"))
        verify_result(args, plan, result)
        append_result_csv(results_file, numeric_result_row(result))
        finished.add(cell)
        print(f"recorded {results_file}: budget={plan.flops_budget:.6g} depth={plan.depth}")


def analyze(args) -> None:
    rows = load_result_csv(args.results_file)
    analysis = analyze_scaling_results(rows, metric=args.metric)
    if not analysis["optimums"]:
        raise RuntimeError("need at least three valid depths for each FLOP budget")
    text = json.dumps(analysis, indent=2)
    print(text)
    if args.output_json is not None:
        Path(args.output_json).parent.mkdir(parents=True, exist_ok=True)
        Path(args.output_json).write_text(text + "\n", encoding="utf-8")
    if args.output_svg is not None:
        write_scaling_svg(args.output_svg, rows, analysis, metric=args.metric)


def validate_run_arguments(args) -> None:
    if (args.eval_batches < 1 or args.num_workers < 0 or args.warmup_steps < 0
            or args.muon_momentum_warmup_iters < 0):
        raise ValueError("evaluation, worker, and warmup values are invalid")
    if not 0 < args.warmup_fraction <= 1:
        raise ValueError("warmup-fraction must be in (0, 1]")
    for name in ("warmdown_ratio", "final_lr_fraction"):
        if not 0 <= getattr(args, name) <= 1:
            raise ValueError(f"{name.replace('_', '-')} must be in [0, 1]")
    if args.max_corpus_epochs <= 0:
        raise ValueError("max-corpus-epochs must be positive")


def main(argv=None) -> None:
    args = parse_args(argv)
    if args.command == "analyze":
        analyze(args)
        return
    if args.command == "run":
        validate_run_arguments(args)
    plans = build_plans(args)
    print_plans(plans)
    if args.command == "plan":
        if args.output_json is not None:
            Path(args.output_json).parent.mkdir(parents=True, exist_ok=True)
            Path(args.output_json).write_text(
                json.dumps([p.to_dict() for p in plans], indent=2) + "\n", encoding="utf-8")
        return
    run_sweep(args, plans)


if __name__ == "__main__":
    main()
