"""Compute-optimal scaling experiments: depth-dialled model shapes, run planning, schedules for
the Muon recipe, and iso-FLOP analysis with a dependency-free SVG report.

Rules and defaults follow the reference planner (ohara/scaling.py:27-751), which in turn follows
nanochat: hidden = round_up(64·depth, 128); FFN = round_up(ceil(8/3·hidden), 256); batch ∝
tokens^0.383 rounded to a power of two; learning rates ∝ √(batch/2^19); weight decay ∝ √(batch)
· (reference tokens / tokens).
"""

from __future__ import annotations

import csv
import html
import math
from collections.abc import Iterable, Mapping, Sequence
from dataclasses import asdict, dataclass
from pathlib import Path

import numpy as np
import torch

from ohara_b200.models.llama import Config, Llama


def _round_up(value: int, multiple: int) -> int:
    if multiple < 1:
        raise ValueError("multiple must be positive")
    return multiple * ((value + multiple - 1) // multiple)


def _nearest_power_of_two(value: float) -> int:
    if value <= 0:
        raise ValueError("value must be positive")
    return 2 ** round(math.log2(value))


def llama_config_for_depth(depth: int, *, vocab_size: int, sequence_length: int = 2_048,
                           aspect_ratio: int = 64, head_dim: int = 128,
                           ffn_multiplier: float = 8 / 3, ffn_multiple_of: int = 256,
                           dropout: float = 0.0, weight_tying: bool = False) -> Config:
    """Every Llama shape from the one scaling dial, depth."""
    if depth < 1:
        raise ValueError("depth must be positive")
    if vocab_size < 2 or sequence_length < 2:
        raise ValueError("vocab_size and sequence_length must be at least 2")
    if aspect_ratio < 1 or head_dim < 2 or head_dim % 2:
        raise ValueError("aspect_ratio must be positive and head_dim must be positive and even")
    if ffn_multiplier <= 0:
        raise ValueError("ffn_multiplier must be positive")
    hidden = _round_up(depth * aspect_ratio, head_dim)
    heads = hidden // head_dim
    return Config(
        vocab_size=vocab_size, max_sequence_length=sequence_length, hidden_size=hidden,
        intermediate_size=_round_up(math.ceil(ffn_multiplier * hidden), ffn_multiple_of),
        num_attention_heads=heads, num_key_value_heads=heads, num_hidden_layers=depth,
        dropout=dropout, multiple_of=ffn_multiple_of, weight_tying=weight_tying,
        init_style="nanochat",
    )


def model_scaling_stats(config: Config) -> tuple[dict[str, int], float]:
    """Parameter groups and FLOPs/token of ``config`` without allocating it (meta device)."""
    with torch.device("meta"):
        model = Llama(config)
    return model.num_scaling_params(), model.estimate_flops(config.max_sequence_length)


@dataclass(frozen=True)
class ScalingPlan:
    depth: int
    hidden_size: int
    intermediate_size: int
    num_heads: int
    sequence_length: int
    params_token_embeddings: int
    params_lm_head: int
    params_transformer: int
    params_norms_and_scalars: int
    params_total: int
    params_effective: int
    flops_per_token: float
    flops_budget: float
    total_batch_size: int
    device_batch_size: int
    world_size: int
    grad_accum_steps: int
    num_iterations: int
    tokens_trained: int
    actual_training_flops: float
    tokens_per_effective_param: float
    learning_rate: float
    matrix_learning_rate: float
    embedding_learning_rate: float
    unembedding_learning_rate: float
    scalar_learning_rate: float
    weight_decay: float

    def to_dict(self) -> dict[str, int | float]:
        return asdict(self)


def plan_scaling_run(depth: int, *, vocab_size: int, flops_budget: float | None = None,
                     target_param_data_ratio: float | None = None, sequence_length: int = 2_048,
                     device_batch_size: int = 32, world_size: int = 1,
                     total_batch_size: int | None = None, aspect_ratio: int = 64,
                     head_dim: int = 128, ffn_multiplier: float = 8 / 3,
                     ffn_multiple_of: int = 256, reference_depth: int = 12,
                     reference_batch_size: int = 2**19, reference_tokens_per_param: float = 12.0,
                     batch_exponent: float = 0.383, base_learning_rate: float = 0.02,
                     base_embedding_learning_rate: float = 0.3,
                     base_unembedding_learning_rate: float = 0.008,
                     base_scalar_learning_rate: float = 0.5,
                     base_weight_decay: float = 0.28) -> ScalingPlan:
    """Plan one run at a fixed FLOP budget, or at a fixed tokens-per-parameter ratio."""
    if flops_budget is None and target_param_data_ratio is None:
        raise ValueError("provide flops_budget or target_param_data_ratio")
    if flops_budget is not None and flops_budget <= 0:
        raise ValueError("flops_budget must be positive")
    if target_param_data_ratio is not None and target_param_data_ratio <= 0:
        raise ValueError("target_param_data_ratio must be positive")
    if device_batch_size < 1 or world_size < 1:
        raise ValueError("device_batch_size and world_size must be positive")
    if reference_batch_size < 1 or reference_tokens_per_param <= 0:
        raise ValueError("reference scaling values must be positive")
    rates = (base_learning_rate, base_embedding_learning_rate, base_unembedding_learning_rate,
             base_scalar_learning_rate)
    if any(v <= 0 for v in rates) or base_weight_decay < 0:
        raise ValueError("optimizer values are invalid")

    shape = dict(vocab_size=vocab_size, sequence_length=sequence_length, aspect_ratio=aspect_ratio,
                 head_dim=head_dim, ffn_multiplier=ffn_multiplier, ffn_multiple_of=ffn_multiple_of)
    config = llama_config_for_depth(depth, **shape)
    counts, flops_per_token = model_scaling_stats(config)
    ref_counts, _ = model_scaling_stats(llama_config_for_depth(reference_depth, **shape))
    ref_tokens = reference_tokens_per_param * ref_counts["effective"]
    nominal_tokens = reference_tokens_per_param * counts["effective"]

    micro_tokens = device_batch_size * sequence_length * world_size
    if total_batch_size is None:
        total_batch_size = _nearest_power_of_two(
            reference_batch_size * (nominal_tokens / ref_tokens) ** batch_exponent
        )
        if total_batch_size < micro_tokens:
            raise ValueError(
                f"the scaling law predicts total_batch_size={total_batch_size:,} tokens for "
                f"depth={depth}, but one distributed micro-batch is already {micro_tokens:,} "
                "tokens (device_batch_size * sequence_length * world_size). Reduce "
                "device_batch_size or world_size for this depth, or pass an explicit "
                "total_batch_size."
            )
    elif total_batch_size < micro_tokens:
        raise ValueError("total_batch_size is smaller than one distributed micro-batch")
    if total_batch_size % micro_tokens:
        raise ValueError("total_batch_size must divide into whole distributed micro-batches")

    if flops_budget is not None:
        iterations = max(1, round(flops_budget / (flops_per_token * total_batch_size)))
        budget = flops_budget
    else:
        # Never overshoot the requested token horizon just to land on a whole step.
        iterations = max(1, int(target_param_data_ratio * counts["effective"] // total_batch_size))
        budget = flops_per_token * total_batch_size * iterations
    tokens = total_batch_size * iterations
    lr_scale = math.sqrt(total_batch_size / reference_batch_size)
    matrix_lr = base_learning_rate * lr_scale
    return ScalingPlan(
        depth=depth, hidden_size=config.hidden_size, intermediate_size=config.intermediate_size,
        num_heads=config.num_attention_heads, sequence_length=sequence_length,
        params_token_embeddings=counts["token_embeddings"], params_lm_head=counts["lm_head"],
        params_transformer=counts["transformer_matrices"],
        params_norms_and_scalars=counts["norms_and_scalars"], params_total=counts["total"],
        params_effective=counts["effective"], flops_per_token=flops_per_token, flops_budget=budget,
        total_batch_size=total_batch_size, device_batch_size=device_batch_size,
        world_size=world_size, grad_accum_steps=total_batch_size // micro_tokens,
        num_iterations=iterations, tokens_trained=tokens,
        actual_training_flops=flops_per_token * tokens,
        tokens_per_effective_param=tokens / counts["effective"], learning_rate=matrix_lr,
        matrix_learning_rate=matrix_lr,
        embedding_learning_rate=base_embedding_learning_rate * lr_scale,
        unembedding_learning_rate=base_unembedding_learning_rate * lr_scale,
        scalar_learning_rate=base_scalar_learning_rate * lr_scale,
        weight_decay=base_weight_decay * lr_scale * (ref_tokens / nominal_tokens),
    )


# --------------------------------------------------------------------------------------------------
# Schedules (trainer iterations are 1-based; these evaluate the 0-based step `iteration - 1`)
# --------------------------------------------------------------------------------------------------
def _check_iteration(iteration: int, max_iters: int) -> None:
    if not 0 <= iteration <= max_iters:
        raise ValueError("iteration must be in [0, max_iters]")


@dataclass(frozen=True)
class WarmupStableDecayScheduler:
    """Linear warmup, constant plateau, linear decay to ``final_lr_fraction`` over the last
    ``warmdown_ratio`` of training."""

    learning_rate: float
    max_iters: int
    warmup_iters: int = 40
    warmdown_ratio: float = 0.65
    final_lr_fraction: float = 0.05

    def __post_init__(self) -> None:
        if self.learning_rate <= 0 or self.max_iters < 1:
            raise ValueError("learning_rate and max_iters must be positive")
        if self.warmup_iters < 0:
            raise ValueError("warmup_iters cannot be negative")
        if not 0 <= self.warmdown_ratio <= 1:
            raise ValueError("warmdown_ratio must be in [0, 1]")
        if not 0 <= self.final_lr_fraction <= 1:
            raise ValueError("final_lr_fraction must be in [0, 1]")

    def __call__(self, iteration: int) -> float:
        _check_iteration(iteration, self.max_iters)
        if iteration == 0:
            return 0.0 if self.warmup_iters else self.learning_rate
        step = iteration - 1
        if self.warmup_iters and step < self.warmup_iters:
            return self.learning_rate * (step + 1) / self.warmup_iters
        decay_steps = round(self.warmdown_ratio * self.max_iters)
        if decay_steps == 0 or step <= self.max_iters - decay_steps:
            return self.learning_rate
        left = (self.max_iters - step) / decay_steps
        return self.learning_rate * (left + (1 - left) * self.final_lr_fraction)


@dataclass(frozen=True)
class MuonMomentumScheduler:
    """Momentum 0.85 → 0.97 over the warmup, held, then → 0.90 over the warmdown window."""

    max_iters: int
    warmdown_ratio: float = 0.65
    warmup_iters: int = 400
    initial_momentum: float = 0.85
    peak_momentum: float = 0.97
    final_momentum: float = 0.90

    def __post_init__(self) -> None:
        if self.max_iters < 1 or self.warmup_iters < 0:
            raise ValueError("max_iters must be positive and warmup_iters non-negative")
        if not 0 <= self.warmdown_ratio <= 1:
            raise ValueError("warmdown_ratio must be in [0, 1]")
        if any(not 0 <= m < 1 for m in (self.initial_momentum, self.peak_momentum, self.final_momentum)):
            raise ValueError("momentum values must be in [0, 1)")

    def __call__(self, iteration: int) -> float:
        _check_iteration(iteration, self.max_iters)
        step = max(0, iteration - 1)
        decay_steps = round(self.warmdown_ratio * self.max_iters)
        decay_start = self.max_iters - decay_steps
        if self.warmup_iters and step < self.warmup_iters:
            return self.initial_momentum + (step / self.warmup_iters) * (
                self.peak_momentum - self.initial_momentum)
        if decay_steps and step >= decay_start:
            return self.peak_momentum + ((step - decay_start) / decay_steps) * (
                self.final_momentum - self.peak_momentum)
        return self.peak_momentum


@dataclass(frozen=True)
class CosineWeightDecayScheduler:
    """Cosine decay of Muon's cautious weight decay to zero."""

    weight_decay: float
    max_iters: int

    def __post_init__(self) -> None:
        if self.weight_decay < 0 or self.max_iters < 1:
            raise ValueError("weight_decay must be non-negative and max_iters positive")

    def __call__(self, iteration: int) -> float:
        _check_iteration(iteration, self.max_iters)
        step = max(0, iteration - 1)
        return self.weight_decay * 0.5 * (1.0 + math.cos(math.pi * step / self.max_iters))


# --------------------------------------------------------------------------------------------------
# Results and analysis
# --------------------------------------------------------------------------------------------------
def append_result_csv(path: str | Path, row: Mapping[str, object]) -> None:
    """Append one result row; the header must match the file's existing header exactly."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    fields = list(row)
    if path.exists():
        with open(path, newline="", encoding="utf-8") as handle:
            header = next(csv.reader(handle), [])
        if header != fields:
            raise ValueError("result row does not match the existing CSV schema")
    with open(path, "a", newline="", encoding="utf-8") as handle:
        writer = csv.DictWriter(handle, fieldnames=fields)
        if handle.tell() == 0:
            writer.writeheader()
        writer.writerow(row)


def load_result_csv(path: str | Path) -> list[dict[str, float]]:
    with open(path, newline="", encoding="utf-8") as handle:
        return [{k: float(v) for k, v in row.items()} for row in csv.DictReader(handle)]


def _quadratic_fit(x: Sequence[float], y: Sequence[float]) -> tuple[float, float, float]:
    """Least-squares ``a·x² + b·x + c``."""
    if len(x) != len(y) or len(x) < 3:
        raise ValueError("quadratic fitting requires at least three paired points")
    xs = np.asarray(x, dtype=np.float64)
    design = np.stack([xs**2, xs, np.ones_like(xs)], axis=1)
    if np.linalg.matrix_rank(design) < 3:
        raise ValueError("cannot fit a quadratic to degenerate points")
    a, b, c = np.linalg.lstsq(design, np.asarray(y, dtype=np.float64), rcond=None)[0]
    return float(a), float(b), float(c)


def fit_isoflop_curves(rows: Iterable[Mapping[str, float]], *,
                       metric: str = "val_bpb") -> list[dict[str, float]]:
    """Per FLOP budget: quadratic of the metric in log10(effective params) and its minimum.
    The fit is done around the mean of the x values (better conditioned) and the coefficients are
    shifted back to absolute log10(params). A minimum outside the sampled range falls back to the
    best sampled point (``interior_optimum = 0``)."""
    by_budget: dict[float, list[Mapping[str, float]]] = {}
    for row in rows:
        value = float(row[metric])
        if math.isfinite(value) and value > 0:
            by_budget.setdefault(float(row["flops_budget"]), []).append(row)
    results = []
    for budget in sorted(by_budget):
        group = sorted(by_budget[budget], key=lambda r: float(r["params_effective"]))
        if len(group) < 3:
            continue
        logs = [math.log10(float(r["params_effective"])) for r in group]
        losses = [float(r[metric]) for r in group]
        centre = sum(logs) / len(logs)
        ca, cb, cc = _quadratic_fit([v - centre for v in logs], losses)
        a, b, c = ca, cb - 2 * ca * centre, ca * centre**2 - cb * centre + cc
        vertex = -b / (2 * a) if a > 0 else float("nan")
        interior = a > 0 and logs[0] <= vertex <= logs[-1]
        if interior:
            best_log, best_loss = vertex, a * vertex**2 + b * vertex + c
        else:
            k = min(range(len(losses)), key=losses.__getitem__)
            best_log, best_loss = logs[k], losses[k]
        # tokens follow from budget = flops/token · tokens; flops/token is near-linear in params,
        # so interpolate that rather than the (steep) token count.
        flops_tok = float(np.interp(best_log, logs, [float(r["flops_per_token"]) for r in group]))
        params = 10**best_log
        tokens = budget / flops_tok
        results.append({
            "flops_budget": budget, "params_effective": params, "tokens_trained": tokens,
            "tokens_per_effective_param": tokens / params, metric: best_loss,
            "quadratic_a": a, "quadratic_b": b, "quadratic_c": c,
            "interior_optimum": float(interior),
        })
    return results


def fit_power_law(rows: Sequence[Mapping[str, float]], *, x_key: str, y_key: str) -> dict[str, float]:
    """``y = coefficient · x^exponent`` by least squares in log-log space."""
    if len(rows) < 2:
        raise ValueError("power-law fitting requires at least two points")
    x = np.log10([float(r[x_key]) for r in rows])
    y = np.log10([float(r[y_key]) for r in rows])
    if np.ptp(x) == 0:
        raise ValueError("power-law x values must not all match")
    exponent, intercept = np.polyfit(x, y, 1)
    residual = float(np.sum((y - (intercept + exponent * x)) ** 2))
    total = float(np.sum((y - y.mean()) ** 2))
    r2 = 1.0 if total == 0 and residual == 0 else 1 - residual / total
    return {"coefficient": float(10**intercept), "exponent": float(exponent), "r_squared": r2}


def analyze_scaling_results(rows: Sequence[Mapping[str, float]], *,
                            metric: str = "val_bpb") -> dict[str, object]:
    optimums = fit_isoflop_curves(rows, metric=metric)
    analysis: dict[str, object] = {"metric": metric, "optimums": optimums}
    interior = [o for o in optimums if o["interior_optimum"] == 1.0]
    analysis["num_interior_optimums"] = len(interior)
    if len(interior) >= 2:
        analysis["optimal_params_power_law"] = fit_power_law(
            interior, x_key="flops_budget", y_key="params_effective")
        analysis["optimal_tokens_power_law"] = fit_power_law(
            interior, x_key="flops_budget", y_key="tokens_trained")
    else:
        analysis["power_law_warning"] = (
            "Need interior iso-FLOP minima for at least two compute budgets; "
            "expand the depth grid before interpreting scaling exponents."
        )
    return analysis


class _Panel:
    """One plot area of the SVG with linear axes over given data bounds."""

    def __init__(self, left: float, top: float, width: float, height: float, title: str,
                 xlabel: str, ylabel: str, xs: Sequence[float], ys: Sequence[float]) -> None:
        self.left, self.top, self.width, self.height = left, top, width, height
        self.title, self.xlabel, self.ylabel = title, xlabel, ylabel
        self.x0, self.x1 = self._pad(xs)
        self.y0, self.y1 = self._pad(ys)

    @staticmethod
    def _pad(values: Sequence[float], frac: float = 0.08) -> tuple[float, float]:
        lo, hi = min(values), max(values)
        if lo == hi:
            return lo - 0.5, hi + 0.5
        extra = (hi - lo) * frac
        return lo - extra, hi + extra

    def xy(self, x: float, y: float) -> tuple[float, float]:
        px = self.left + (x - self.x0) / (self.x1 - self.x0) * self.width
        py = self.top + self.height - (y - self.y0) / (self.y1 - self.y0) * self.height
        return px, py

    def frame(self) -> list[str]:
        out = [f'<text class="title" x="{self.left}" y="{self.top - 14}">{html.escape(self.title)}</text>']
        for i in range(5):
            fx = self.x0 + (self.x1 - self.x0) * i / 4
            fy = self.y0 + (self.y1 - self.y0) * i / 4
            gx, _ = self.xy(fx, self.y0)
            _, gy = self.xy(self.x0, fy)
            out.append(f'<line class="grid" x1="{gx:.1f}" y1="{self.top}" x2="{gx:.1f}" y2="{self.top + self.height}"/>')
            out.append(f'<line class="grid" x1="{self.left}" y1="{gy:.1f}" x2="{self.left + self.width}" y2="{gy:.1f}"/>')
            out.append(f'<text class="label" text-anchor="middle" x="{gx:.1f}" y="{self.top + self.height + 16}">{fx:.2f}</text>')
            out.append(f'<text class="label" text-anchor="end" x="{self.left - 6}" y="{gy + 4:.1f}">{fy:.3g}</text>')
        out.append(f'<rect class="axis" fill="none" x="{self.left}" y="{self.top}" width="{self.width}" height="{self.height}"/>')
        out.append(f'<text class="label" text-anchor="middle" x="{self.left + self.width / 2}" y="{self.top + self.height + 34}">{html.escape(self.xlabel)}</text>')
        out.append(f'<text class="label" text-anchor="middle" transform="rotate(-90 {self.left - 44} {self.top + self.height / 2})" x="{self.left - 44}" y="{self.top + self.height / 2}">{html.escape(self.ylabel)}</text>')
        return out


def write_scaling_svg(path: str | Path, rows: Sequence[Mapping[str, float]],
                      analysis: Mapping[str, object], *, metric: str = "val_bpb") -> None:
    """Three panels: iso-FLOP curves with fitted parabolas, optimal parameters vs compute, optimal
    tokens vs compute (both log-log with the fitted power laws). Plain SVG text, no plotting
    library."""
    optimums = list(analysis.get("optimums", []))
    if not optimums:
        raise ValueError("analysis contains no iso-FLOP optimums")
    colors = ("#2563eb", "#059669", "#d97706", "#dc2626", "#7c3aed", "#0891b2")
    usable = [r for r in rows if math.isfinite(float(r[metric])) and float(r[metric]) > 0]
    budgets = sorted({float(o["flops_budget"]) for o in optimums})
    svg = [
        '<svg xmlns="http://www.w3.org/2000/svg" width="1260" height="420" viewBox="0 0 1260 420">',
        '<rect width="100%" height="100%" fill="white"/>',
        '<style>text{font-family:system-ui,sans-serif;fill:#111827}.title{font-size:16px;'
        'font-weight:600}.label{font-size:12px;fill:#4b5563}.axis{stroke:#9ca3af;stroke-width:1}'
        '.grid{stroke:#e5e7eb;stroke-width:1}</style>',
    ]
    log_p = [math.log10(float(r["params_effective"])) for r in usable]
    p1 = _Panel(65, 55, 340, 290, f"Iso-FLOP curves ({metric})", "log10 effective parameters",
                metric, log_p, [float(r[metric]) for r in usable])
    svg += p1.frame()
    for index, budget in enumerate(budgets):
        color = colors[index % len(colors)]
        optimum = next(o for o in optimums if float(o["flops_budget"]) == budget)
        group = sorted((r for r in usable if float(r["flops_budget"]) == budget),
                       key=lambda r: float(r["params_effective"]))
        xs = [math.log10(float(r["params_effective"])) for r in group]
        a, b, c = (float(optimum[k]) for k in ("quadratic_a", "quadratic_b", "quadratic_c"))
        curve = []
        for i in range(41):
            x = xs[0] + (xs[-1] - xs[0]) * i / 40
            y = min(max(a * x * x + b * x + c, p1.y0), p1.y1)
            curve.append("{:.1f},{:.1f}".format(*p1.xy(x, y)))
        svg.append(f'<polyline fill="none" stroke="{color}" stroke-width="1.5" points="{" ".join(curve)}"/>')
        for row, x in zip(group, xs):
            cx, cy = p1.xy(x, float(row[metric]))
            svg.append(f'<circle cx="{cx:.1f}" cy="{cy:.1f}" r="3.5" fill="{color}"/>')
        ox, oy = p1.xy(math.log10(float(optimum["params_effective"])), float(optimum[metric]))
        svg.append(f'<path d="M{ox - 5:.1f},{oy:.1f} L{ox:.1f},{oy - 5:.1f} L{ox + 5:.1f},{oy:.1f} '
                   f'L{ox:.1f},{oy + 5:.1f} Z" fill="none" stroke="{color}" stroke-width="2"/>')
        svg.append(f'<text class="label" x="{p1.left + 8}" y="{p1.top + 16 + 14 * index}" '
                   f'fill="{color}">{budget:.1e} FLOPs</text>')

    log_c = [math.log10(float(o["flops_budget"])) for o in optimums]
    for panel_index, (key, title, law_key) in enumerate((
        ("params_effective", "optimal parameters", "optimal_params_power_law"),
        ("tokens_trained", "optimal tokens", "optimal_tokens_power_law"),
    )):
        ys = [math.log10(float(o[key])) for o in optimums]
        panel = _Panel(465 + 400 * panel_index, 55, 340, 290, title, "log10 training FLOPs",
                       f"log10 {key}", log_c, ys)
        svg += panel.frame()
        law = analysis.get(law_key)
        if isinstance(law, Mapping):
            intercept = math.log10(float(law["coefficient"]))
            ends = [panel.xy(x, min(max(intercept + float(law["exponent"]) * x, panel.y0), panel.y1))
                    for x in (min(log_c), max(log_c))]
            svg.append(f'<line x1="{ends[0][0]:.1f}" y1="{ends[0][1]:.1f}" x2="{ends[1][0]:.1f}" '
                       f'y2="{ends[1][1]:.1f}" stroke="#111827" stroke-dasharray="5 4"/>')
            svg.append(f'<text class="label" x="{panel.left + 8}" y="{panel.top + 16}">'
                       f'exponent {float(law["exponent"]):.3f}, R² {float(law["r_squared"]):.3f}</text>')
        for index, (optimum, x, y) in enumerate(zip(optimums, log_c, ys)):
            cx, cy = panel.xy(x, y)
            hollow = float(optimum["interior_optimum"]) != 1.0
            color = colors[index % len(colors)]
            svg.append(f'<circle cx="{cx:.1f}" cy="{cy:.1f}" r="4.5" stroke="{color}" stroke-width="2" '
                       f'fill="{"white" if hollow else color}"/>')
    if "power_law_warning" in analysis:
        svg.append(f'<text class="label" x="465" y="400">{html.escape(str(analysis["power_law_warning"]))}</text>')
    svg.append("</svg>")
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text("\n".join(svg) + "\n", encoding="utf-8")
