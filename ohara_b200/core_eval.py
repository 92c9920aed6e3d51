"""CORE in-context-learning evaluation (the DCLM / nanochat "core metric").

Three task types, all scored by next-token losses of one forward pass per example:

* ``multiple_choice`` — one prompt per choice; choices share a prefix, the scored span starts at
  the first token where they differ; lowest mean loss wins.
* ``schema`` — one prompt per context option, shared continuation; the scored span is the common
  suffix.
* ``language_modeling`` — context vs context+continuation; correct iff every continuation token is
  the argmax prediction. With BPE the context may not tokenise to an exact prefix, so scoring
  starts at the last genuinely shared token.

Few-shot examples are drawn with ``random.Random(1234 + idx)``; prompts longer than the model's
context are cropped from the left (an example whose answer span is cropped away counts as wrong);
examples are striped over ranks and correctness all-reduced; accuracies are centred against the
task's random baseline and averaged. Behaviour follows ohara/core_eval.py:50-367.
"""

from __future__ import annotations

import csv
import io
import json
import random
import shutil
import tempfile
import zipfile
from dataclasses import dataclass
from pathlib import Path
from urllib.request import urlopen

import torch
import torch.distributed as dist

EVAL_BUNDLE_URL = "https://karpathy-public.s3.us-west-2.amazonaws.com/eval_bundle.zip"


# -- tokenizer helpers ---------------------------------------------------------------------------
def _get_bos_token_id(tokenizer) -> int:
    getter = getattr(tokenizer, "get_bos_token_id", None)
    if callable(getter) and getter() is not None:
        return int(getter())
    for name in ("bos_token_id", "eos_token_id"):
        value = getattr(tokenizer, name, None)
        if value is not None:
            return int(value)
    convert = getattr(tokenizer, "convert_tokens_to_ids", None)
    if callable(convert):
        for token in ("<|bos|>", "<|endoftext|>"):
            token_id = convert(token)
            if token_id is not None and token_id != -1:
                return int(token_id)
    raise ValueError("Failed to infer BOS token id from tokenizer")


def _encode_text(tokenizer, text: str) -> list[int]:
    if not hasattr(tokenizer, "encode"):
        raise TypeError("Tokenizer must provide an encode method")
    try:
        return list(tokenizer.encode(text, add_special_tokens=False))
    except TypeError:
        return list(tokenizer.encode(text))


def _encode_with_bos(tokenizer, text: str) -> list[int]:
    return [_get_bos_token_id(tokenizer)] + _encode_text(tokenizer, text)


# -- prompt rendering -------------------------------------------------------------------------------
def render_prompts_mc(item, continuation_delimiter, fewshot_examples=None):
    shots = "".join(
        f"{ex['query']}{continuation_delimiter}{ex['choices'][ex['gold']]}\n\n"
        for ex in (fewshot_examples or [])
    )
    return [f"{shots}{item['query']}{continuation_delimiter}{choice}" for choice in item["choices"]]


def render_prompts_schema(item, continuation_delimiter, fewshot_examples=None):
    shots = "".join(
        f"{ex['context_options'][ex['gold']]}{continuation_delimiter}{ex['continuation']}\n\n"
        for ex in (fewshot_examples or [])
    )
    return [f"{shots}{option}{continuation_delimiter}{item['continuation']}"
            for option in item["context_options"]]


def render_prompts_lm(item, continuation_delimiter, fewshot_examples=None):
    shots = "".join(
        f"{ex['context'].strip()}{continuation_delimiter}{ex['continuation']}\n\n"
        for ex in (fewshot_examples or [])
    )
    without = f"{shots}{item['context'].strip()}{continuation_delimiter}".strip()
    return [without, f"{without}{item['continuation']}"]


def find_common_length(token_sequences, direction: str = "left") -> int:
    """Length of the common prefix (``left``) or suffix (``right``) of the sequences."""
    if direction not in ("left", "right"):
        raise ValueError(f"Unsupported direction: {direction}")
    shortest = min(len(seq) for seq in token_sequences)
    for offset in range(shortest):
        pos = offset if direction == "left" else -1 - offset
        first = token_sequences[0][pos]
        if any(seq[pos] != first for seq in token_sequences):
            return offset
    return shortest


def stack_sequences(tokens, pad_token_id: int) -> torch.Tensor:
    width = max(len(row) for row in tokens)
    out = torch.full((len(tokens), width), pad_token_id, dtype=torch.long)
    for i, row in enumerate(tokens):
        out[i, : len(row)] = torch.tensor(row, dtype=torch.long)
    return out


def batch_sequences_mc(tokenizer, prompts):
    tokens = [_encode_with_bos(tokenizer, p) for p in prompts]
    start = find_common_length(tokens, "left")
    return tokens, [start] * len(tokens), [len(t) for t in tokens]


def batch_sequences_schema(tokenizer, prompts):
    tokens = [_encode_with_bos(tokenizer, p) for p in prompts]
    suffix = find_common_length(tokens, "right")
    ends = [len(t) for t in tokens]
    return tokens, [e - suffix for e in ends], ends


def batch_sequences_lm(tokenizer, prompts):
    tokens = [_encode_with_bos(tokenizer, p) for p in prompts]
    without, full = tokens
    start = find_common_length(tokens, "left")
    if start >= len(full):
        raise ValueError(
            "language-modeling continuation is empty in token space: "
            f"context={len(without)} tokens, full={len(full)} tokens"
        )
    return [full], [start], [len(full)]


@dataclass(frozen=True)
class _TaskType:
    render: callable
    batch: callable


_TASK_TYPES = {
    "multiple_choice": _TaskType(render_prompts_mc, batch_sequences_mc),
    "schema": _TaskType(render_prompts_schema, batch_sequences_schema),
    "language_modeling": _TaskType(render_prompts_lm, batch_sequences_lm),
}

# Context-window attribute names used by this package and by Hugging Face models.
_MAX_SEQ_LEN_ATTRS = ("max_seq_len", "max_sequence_length", "seq_len", "sequence_len",
                      "n_positions", "max_position_embeddings")


def infer_model_max_seq_len(model) -> int | None:
    holders = [model, getattr(model, "config", None)]
    inner = getattr(model, "model", None)
    if inner is not None:
        holders += [inner, getattr(inner, "config", None)]
    for holder in holders:
        if holder is None:
            continue
        for name in _MAX_SEQ_LEN_ATTRS:
            value = getattr(holder, name, None)
            if isinstance(value, int) and value > 0:
                return value
    return None


@torch.no_grad()
def forward_model(model, input_ids):
    """Per-position next-token losses (last column NaN) and argmax predictions."""
    outputs = model(input_ids)
    logits = outputs.logits if hasattr(outputs, "logits") else outputs
    batch, seq = input_ids.shape
    targets = torch.roll(input_ids, shifts=-1, dims=1)
    losses = torch.nn.functional.cross_entropy(
        logits.float().view(batch * seq, -1), targets.view(batch * seq), reduction="none"
    ).view(batch, seq)
    losses[:, -1] = float("nan")
    return losses, logits.argmax(dim=-1)


@torch.no_grad()
def evaluate_example(idx, model, tokenizer, data, device, task_meta) -> bool:
    item = data[idx]
    kind = task_meta["task_type"]
    if kind not in _TASK_TYPES:
        raise ValueError(f"Unsupported task type: {kind}")
    shots = []
    if task_meta["num_fewshot"] > 0:
        pool = [i for i in range(len(data)) if i != idx]
        shots = [data[i] for i in random.Random(1234 + idx).sample(pool, task_meta["num_fewshot"])]
    task = _TASK_TYPES[kind]
    prompts = task.render(item, task_meta["continuation_delimiter"], shots)
    tokens, starts, ends = task.batch(tokenizer, prompts)

    limit = infer_model_max_seq_len(model)
    if limit is not None:
        cropped = []
        for row, start, end in zip(tokens, starts, ends):
            cut = max(len(row) - limit, 0)
            if cut and (start - cut < 1 or end - cut < 1):
                # the answer span, or the token that predicts its first token, was cropped away
                return False
            cropped.append((row[cut:], start - cut, end - cut))
        tokens, starts, ends = (list(x) for x in zip(*cropped))

    input_ids = stack_sequences(tokens, _get_bos_token_id(tokenizer)).to(device)
    losses, predictions = forward_model(model, input_ids)
    if kind == "language_modeling":
        start, end = starts[0], ends[0]
        return bool(torch.all(predictions[0, start - 1 : end - 1] == input_ids[0, start:end]).item())
    means = [losses[r, s - 1 : e - 1].mean().item() for r, (s, e) in enumerate(zip(starts, ends))]
    return means.index(min(means)) == item["gold"]


def evaluate_task(model, tokenizer, data, device, task_meta) -> float:
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    correct = torch.zeros(len(data), dtype=torch.float32, device=device)
    for idx in range(rank, len(data), world):
        correct[idx] = float(evaluate_example(idx, model, tokenizer, data, device, task_meta))
    if world > 1:
        dist.barrier()
        dist.all_reduce(correct, op=dist.ReduceOp.SUM)
    return correct.mean().item()


def evaluate_core_from_bundle(model, tokenizer, device, eval_bundle_dir, max_per_task: int = -1):
    import yaml

    bundle = Path(eval_bundle_dir)
    with open(bundle / "core.yaml", encoding="utf-8") as handle:
        tasks = yaml.safe_load(handle)["icl_tasks"]
    with open(bundle / "eval_meta_data.csv", encoding="utf-8") as handle:
        baselines = {row["Eval Task"]: float(row["Random baseline"]) for row in csv.DictReader(handle)}
    results, centered = {}, {}
    for task in tasks:
        label = task["label"]
        meta = {
            "task_type": task["icl_task_type"],
            "dataset_uri": task["dataset_uri"],
            "num_fewshot": task["num_fewshot"][0],
            "continuation_delimiter": task.get("continuation_delimiter", " "),
        }
        with open(bundle / "eval_data" / meta["dataset_uri"], encoding="utf-8") as handle:
            data = [json.loads(line.strip()) for line in handle]
        random.Random(1337).shuffle(data)
        if max_per_task > 0:
            data = data[:max_per_task]
        accuracy = evaluate_task(model, tokenizer, data, device, meta)
        results[label] = accuracy
        floor = 0.01 * baselines[label]
        centered[label] = (accuracy - floor) / (1.0 - floor)
    return {"results": results, "centered_results": centered,
            "core_metric": sum(centered.values()) / len(centered)}


def _download_eval_bundle(eval_bundle_dir: Path, bundle_url: str) -> None:
    eval_bundle_dir.parent.mkdir(parents=True, exist_ok=True)
    with urlopen(bundle_url) as response:
        payload = response.read()
    with tempfile.TemporaryDirectory() as scratch:
        with zipfile.ZipFile(io.BytesIO(payload), "r") as archive:
            archive.extractall(scratch)
        if eval_bundle_dir.exists():
            shutil.rmtree(eval_bundle_dir)
        shutil.move(str(Path(scratch) / "eval_bundle"), str(eval_bundle_dir))


def evaluate_core(model, tokenizer, device, *, max_per_task: int = -1,
                  eval_bundle_dir: str | Path = "./eval_bundle", bundle_url: str = EVAL_BUNDLE_URL):
    bundle = Path(eval_bundle_dir)
    if not bundle.exists():
        _download_eval_bundle(bundle, bundle_url)
    return evaluate_core_from_bundle(model=model, tokenizer=tokenizer, device=device,
                                     eval_bundle_dir=bundle, max_per_task=max_per_task)
