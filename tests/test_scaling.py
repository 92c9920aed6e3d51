"""Scaling planner, schedules and iso-FLOP analysis (reference suite: tests/test_scaling.py:21-127),
plus the sweep driver in examples/scaling_laws.py."""

from __future__ import annotations

import math

import pytest

from ohara_b200.models.llama import Llama
from ohara_b200.scaling import (
    CosineWeightDecayScheduler,
    MuonMomentumScheduler,
    WarmupStableDecayScheduler,
    analyze_scaling_results,
    append_result_csv,
    fit_power_law,
    llama_config_for_depth,
    load_result_csv,
    model_scaling_stats,
    plan_scaling_run,
    write_scaling_svg,
)
from test_data import load_example

SMALL = dict(vocab_size=512, sequence_length=64, aspect_ratio=16, head_dim=16, ffn_multiple_of=16)


def test_depth_sets_every_shape():
    config = llama_config_for_depth(6, **SMALL)
    assert config.hidden_size == 96 and config.num_attention_heads == 6
    assert config.num_hidden_layers == 6 and config.intermediate_size == 256
    assert not config.weight_tying and config.init_style == "nanochat"
    odd = llama_config_for_depth(5, vocab_size=512, sequence_length=64, aspect_ratio=10, head_dim=16)
    assert odd.hidden_size == 64, "width is rounded up to whole heads"
    counts, flops = model_scaling_stats(config)
    model = Llama(config)
    assert counts["total"] == sum(p.numel() for p in model.parameters())
    assert counts["effective"] == counts["transformer_matrices"] + counts["lm_head"]
    assert flops == model.estimate_flops(64)
    for bad in (dict(depth=0), dict(depth=2, head_dim=7), dict(depth=2, ffn_multiplier=0)):
        depth = bad.pop("depth")
        with pytest.raises(ValueError):
            llama_config_for_depth(depth, **{**SMALL, **bad})


def test_fixed_flop_plan_adds_up():
    plan = plan_scaling_run(4, flops_budget=2e12, device_batch_size=2, world_size=2,
                            reference_depth=4, reference_batch_size=1024, **SMALL)
    assert plan.total_batch_size == 1024, "the reference depth gets the reference batch"
    assert plan.grad_accum_steps == 1024 // (2 * 64 * 2)
    assert plan.tokens_trained == plan.total_batch_size * plan.num_iterations
    assert math.isclose(plan.actual_training_flops, plan.flops_per_token * plan.tokens_trained)
    assert abs(plan.actual_training_flops - 2e12) <= plan.flops_per_token * plan.total_batch_size
    assert math.isclose(plan.matrix_learning_rate, 0.02) and math.isclose(plan.weight_decay, 0.28)
    deeper = plan_scaling_run(8, flops_budget=2e12, device_batch_size=2, reference_depth=4,
                              reference_batch_size=1024, **SMALL)
    assert deeper.total_batch_size > plan.total_batch_size
    assert deeper.matrix_learning_rate > plan.matrix_learning_rate
    assert deeper.weight_decay < plan.weight_decay
    assert set(plan.to_dict()) >= {"depth", "hidden_size", "num_iterations", "weight_decay"}
    with pytest.raises(ValueError, match="flops_budget or target_param_data_ratio"):
        plan_scaling_run(4, **SMALL)
    with pytest.raises(ValueError, match="micro-batch"):
        plan_scaling_run(4, flops_budget=1e12, total_batch_size=64, device_batch_size=2, **SMALL)
    with pytest.raises(ValueError, match="whole distributed micro-batches"):
        plan_scaling_run(4, flops_budget=1e12, total_batch_size=200, device_batch_size=2, **SMALL)


def test_token_ratio_plan_never_overshoots():
    plan = plan_scaling_run(4, target_param_data_ratio=3.0, device_batch_size=2,
                            total_batch_size=1024, **SMALL)
    assert plan.tokens_trained <= 3.0 * plan.params_effective
    assert plan.tokens_trained + plan.total_batch_size > 3.0 * plan.params_effective or plan.num_iterations == 1
    assert math.isclose(plan.flops_budget, plan.actual_training_flops)


def test_schedules_hit_their_boundaries():
    lr = WarmupStableDecayScheduler(learning_rate=1.0, max_iters=100, warmup_iters=10,
                                    warmdown_ratio=0.5, final_lr_fraction=0.1)
    assert lr(0) == 0.0 and math.isclose(lr(1), 0.1) and lr(10) == 1.0 and lr(50) == 1.0
    assert lr(51) == 1.0 and lr(52) < 1.0 and lr(100) > 0.1 and lr(100) < 0.2
    assert WarmupStableDecayScheduler(learning_rate=2.0, max_iters=10, warmup_iters=0,
                                      warmdown_ratio=0.0)(10) == 2.0
    momentum = MuonMomentumScheduler(max_iters=100, warmdown_ratio=0.5, warmup_iters=10)
    assert momentum(1) == 0.85 and math.isclose(momentum(11), 0.97) and momentum(40) == 0.97
    assert 0.90 < momentum(100) < 0.97
    decay = CosineWeightDecayScheduler(weight_decay=0.2, max_iters=100)
    assert decay(1) == 0.2 and math.isclose(decay(51), 0.1) and decay(100) < 1e-3
    for schedule in (lr, momentum, decay):
        with pytest.raises(ValueError):
            schedule(101)
    for bad in (dict(learning_rate=0.0, max_iters=10), dict(learning_rate=1.0, max_iters=10, warmdown_ratio=2)):
        with pytest.raises(ValueError):
            WarmupStableDecayScheduler(**bad)


def _synthetic_rows():
    """Loss surfaces with a known interior optimum that moves as budget^0.5."""
    rows = []
    for budget in (1e15, 4e15, 1.6e16):
        best = 1e6 * math.sqrt(budget / 1e15)
        for scale in (0.25, 0.5, 1.0, 2.0, 4.0):
            params = best * scale
            flops_per_token = 6.0 * params
            rows.append({"flops_budget": budget, "depth": round(10 * scale), "params_effective": params,
                         "flops_per_token": flops_per_token, "tokens_trained": budget / flops_per_token,
                         "val_bpb": 1.0 + 0.2 * math.log10(scale) ** 2 - 0.05 * math.log10(budget / 1e15)})
    return rows


def test_csv_round_trip_and_isoflop_fit(tmp_path):
    path = tmp_path / "out" / "results.csv"
    rows = _synthetic_rows()
    for row in rows:
        append_result_csv(path, row)
    with pytest.raises(ValueError, match="schema"):
        append_result_csv(path, {"something": 1.0})
    loaded = load_result_csv(path)
    assert len(loaded) == len(rows) and all(isinstance(v, float) for v in loaded[0].values())

    analysis = analyze_scaling_results(loaded)
    assert analysis["num_interior_optimums"] == 3
    for optimum, budget in zip(analysis["optimums"], (1e15, 4e15, 1.6e16)):
        assert math.isclose(optimum["params_effective"], 1e6 * math.sqrt(budget / 1e15), rel_tol=1e-3)
    assert math.isclose(analysis["optimal_params_power_law"]["exponent"], 0.5, abs_tol=1e-3)
    assert math.isclose(analysis["optimal_tokens_power_law"]["exponent"], 0.5, abs_tol=1e-3)
    assert analysis["optimal_params_power_law"]["r_squared"] > 0.999

    svg = tmp_path / "fit.svg"
    write_scaling_svg(svg, loaded, analysis)
    text = svg.read_text()
    assert text.startswith("<svg") or text.lstrip().startswith("<?xml") or "<svg" in text[:200]
    assert text.count("<circle") >= len(rows)

    monotone = [dict(r, val_bpb=1.0 - 0.1 * math.log10(r["params_effective"])) for r in rows]
    edge = analyze_scaling_results(monotone)
    assert edge["num_interior_optimums"] == 0 and "power_law_warning" in edge
    with pytest.raises(ValueError):
        fit_power_law(rows[:1], x_key="flops_budget", y_key="params_effective")


# -- examples/scaling_laws.py --------------------------------------------------------------------------
def _sweep_args(sweep, tmp_path, *extra):
    return sweep.parse_args([
        "run", "--dry-run", "--depths", "4,6", "--flops-budgets", "1e12", "--vocab-size", "512",
        "--seq-len", "64", "--device-batch-size", "2", "--aspect-ratio", "16", "--head-dim", "16",
        "--ffn-multiple-of", "16", "--reference-depth", "4", "--reference-batch-size", "1024",
        "--results-dir", str(tmp_path / "results"), "--dataset", str(tmp_path / "corpus"), *extra])


def test_sweep_commands_carry_the_plan(tmp_path, capsys):
    sweep = load_example("scaling_laws")
    args = _sweep_args(sweep, tmp_path, "--optimizer", "muonh", "--hypersphere-learning-rate", "0.05")
    plans = sweep.build_plans(args)
    assert [p.depth for p in plans] == [4, 6]
    command = sweep.training_command(args, plans[0], tmp_path / "r.json")
    option = lambda name: command[command.index(f"--{name}") + 1]  # noqa: E731
    assert option("num-layers") == "4" and option("hidden-size") == str(plans[0].hidden_size)
    assert option("max-iters") == option("eval-every") == str(plans[0].num_iterations)
    assert option("optimizer") == "muonh" and option("hypersphere-learning-rate") == "0.05"
    assert float(option("weight-decay")) == plans[0].weight_decay
    assert "--no-weight-tying" in command and "--evaluate-bpb" in command
    assert int(option("warmup-iters")) == sweep.scaled_warmup_iters(40, plans[0].num_iterations, 0.1)
    sweep.run_sweep(args, plans)
    assert capsys.readouterr().out.count("run: ") == 2
    assert not (tmp_path / "results").exists(), "a dry run writes nothing"


def test_sweep_guards(tmp_path):
    sweep = load_example("scaling_laws")
    args = _sweep_args(sweep, tmp_path)
    plans = sweep.build_plans(args)
    corpus = tmp_path / "corpus"
    corpus.mkdir()
    sweep.check_corpus_epoch_budget(args, plans)  # no stats file: nothing to check
    (corpus / "stats.train.json").write_text('{"tokens": 100}')
    with pytest.raises(ValueError, match="repeat the staged corpus"):
        sweep.check_corpus_epoch_budget(args, plans)
    args.allow_repeated_epochs = True
    sweep.check_corpus_epoch_budget(args, plans)

    results = tmp_path / "results"
    sweep.prepare_results_manifest(args, results)
    sweep.prepare_results_manifest(args, results)  # same settings: accepted
    args.seed = 7
    with pytest.raises(ValueError, match="seed"):
        sweep.prepare_results_manifest(args, results)

    plan = plans[0]
    good = {"params_effective": plan.params_effective, "total_batch_size": plan.total_batch_size,
            "optimizer": "muon", "optimizer_muon": 1.0, "initialization_nanochat": 1.0,
            **{name: getattr(plan, name) for name in sweep._PLANNED_FIELDS}}
    sweep.verify_result(args, plan, good)
    for field, wrong in (("params_effective", 1), ("optimizer", "adamw"), ("weight_decay", 9.0),
                         ("initialization_nanochat", 0.0)):
        with pytest.raises(RuntimeError):
            sweep.verify_result(args, plan, {**good, field: wrong})
    assert sweep.numeric_result_row({"a": 1, "b": "muon", "c": True, "d": 2.5}) == {"a": 1, "d": 2.5}
