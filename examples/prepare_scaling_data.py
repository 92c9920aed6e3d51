"""Stage a bounded text corpus on disk for offline scaling sweeps.

    python examples/prepare_scaling_data.py --train-documents 100000 --validation-documents 10000
    python examples/prepare_scaling_data.py --train-file a.jsonl --validation-file b.jsonl

Writes ``train.jsonl`` / ``validation.jsonl`` (one ``{"text": ...}`` per line) and, when a
tokenizer is given, ``stats.{split}.json`` with the exact token count (one boundary token per
document included) so that scaling_laws.py can refuse a sweep whose token horizon would re-read a
corpus that is too small. The stats file name must not start with the split name: the streaming
dataset finds local files by ``{split}*.json*`` and would otherwise train on it. Without a source
override the corpus is NanoChat's ClimbMix shards with its pinned held-out shard.
Flags follow the reference entry point (examples/prepare_scaling_data.py:40-98).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from dataclasses import dataclass
from pathlib import Path
from urllib.parse import urlparse

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

from ohara_b200.tokenizer import get_tokenizer

CLIMBMIX_URL = "https://huggingface.co/datasets/karpathy/climbmix-400b-shuffle/resolve/main"
CLIMBMIX_VALIDATION_SHARD = 6_542
DEFAULT_TOKENIZER = "EleutherAI/gpt-neo-125m"
_BUILDERS = {".txt": "text", ".json": "json", ".jsonl": "json", ".parquet": "parquet"}


def nanochat_climbmix_files(train_shards: int) -> tuple[list[str], str]:
    """The first ``train_shards`` training shards and the pinned validation shard."""
    if not 1 <= train_shards <= CLIMBMIX_VALIDATION_SHARD:
        raise ValueError(f"climbmix train shards must be between 1 and {CLIMBMIX_VALIDATION_SHARD:,}")
    shard = "{}/shard_{:05d}.parquet".format
    return ([shard(CLIMBMIX_URL, i) for i in range(train_shards)],
            shard(CLIMBMIX_URL, CLIMBMIX_VALIDATION_SHARD))


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Stage a bounded text corpus for offline scaling sweeps")
    p.add_argument("--dataset", default=None, help="Hugging Face dataset instead of ClimbMix")
    p.add_argument("--dataset-config", default=None)
    p.add_argument("--text-column", default="text")
    p.add_argument("--train-split", default="train")
    p.add_argument("--validation-split", default="validation")
    p.add_argument("--train-file", action="append", default=None, help="repeatable")
    p.add_argument("--validation-file", action="append", default=None, help="repeatable")
    p.add_argument("--climbmix-train-shards", type=int, default=10)
    p.add_argument("--train-documents", type=int, default=100_000)
    p.add_argument("--validation-documents", type=int, default=10_000)
    p.add_argument("--output-dir", default="./data/scaling_corpus")
    p.add_argument("--force", action="store_true")
    p.add_argument("--skip-existing", action="store_true")
    p.add_argument("--tokenizer", default=DEFAULT_TOKENIZER,
                   help="count tokens while staging (pass an empty string to skip)")
    p.add_argument("--tokenizer-batch-size", type=int, default=256)
    p.add_argument("--tokenizer-local-files-only", action="store_true")
    return p.parse_args()


def count_tokens(tokenizer, texts: list[str]) -> int:
    """Model tokens plus one document-boundary token per document."""
    if callable(tokenizer):
        ids = tokenizer(texts, add_special_tokens=False, return_attention_mask=False,
                        return_token_type_ids=False)["input_ids"]
        return sum(len(row) + 1 for row in ids)
    return sum(len(tokenizer.encode(text, add_special_tokens=False)) + 1 for text in texts)


def _atomic_write_text(path: Path, text: str) -> None:
    temporary = path.with_name(f".{path.name}.tmp-{os.getpid()}")
    try:
        temporary.write_text(text, encoding="utf-8")
        os.replace(temporary, path)
    finally:
        temporary.unlink(missing_ok=True)


def open_stream(*, dataset_name, dataset_config, source_files, source_split):
    from datasets import load_dataset

    if source_files is not None:
        if not source_files:
            raise ValueError("source_files cannot be empty")
        suffixes = {Path(urlparse(src).path).suffix.lower() for src in source_files}
        if len(suffixes) != 1 or not suffixes <= set(_BUILDERS):
            raise ValueError(f"source files must share a supported suffix: {source_files}")
        return load_dataset(path=_BUILDERS[suffixes.pop()], data_files={source_split: source_files},
                            split=source_split, streaming=True)
    if dataset_name is None:
        raise ValueError("dataset_name is required when source_files are not provided")
    extra = {"name": dataset_config} if dataset_config is not None else {}
    return load_dataset(path=dataset_name, split=source_split, streaming=True, **extra)


@dataclass
class Staged:
    documents: int = 0
    utf8_bytes: int = 0
    tokens: int | None = None


def stage_split(*, dataset_name, dataset_config, source_files, source_split, output_split,
                text_column, max_documents, output_dir: Path, force, skip_existing,
                tokenizer=None, tokenizer_batch_size: int = 256, stream=None) -> Staged | None:
    """Copy up to ``max_documents`` usable rows into ``{output_split}.jsonl``; ``None`` when an
    existing file was kept. ``stream`` lets a caller supply rows directly."""
    if max_documents < 1:
        raise ValueError("document limits must be positive")
    if tokenizer_batch_size < 1:
        raise ValueError("tokenizer batch size must be positive")
    target = output_dir / f"{output_split}.jsonl"
    if target.exists() and not force:
        if skip_existing:
            return None
        raise FileExistsError(f"{target} already exists; pass --force to replace it")
    if stream is None:
        stream = open_stream(dataset_name=dataset_name, dataset_config=dataset_config,
                             source_files=source_files, source_split=source_split)
    output_dir.mkdir(parents=True, exist_ok=True)
    done = Staged(tokens=0 if tokenizer is not None else None)
    pending: list[str] = []

    def drain() -> None:
        if pending:
            done.tokens += count_tokens(tokenizer, pending)
            pending.clear()

    temporary = target.with_name(f".{target.name}.tmp-{os.getpid()}")
    try:
        with open(temporary, "w", encoding="utf-8") as handle:
            for row in stream:
                text = row.get(text_column)
                if not isinstance(text, str) or not text:
                    continue
                handle.write(json.dumps({"text": text}, ensure_ascii=False) + "\n")
                done.documents += 1
                done.utf8_bytes += len(text.encode("utf-8"))
                if tokenizer is not None:
                    pending.append(text)
                    if len(pending) >= tokenizer_batch_size:
                        drain()
                if done.documents >= max_documents:
                    break
            if tokenizer is not None:
                drain()
        if done.documents == 0:
            raise RuntimeError(f"no usable text found in split {source_split!r}")
        os.replace(temporary, target)
    finally:
        temporary.unlink(missing_ok=True)
    if done.tokens is not None:
        _atomic_write_text(output_dir / f"stats.{output_split}.json",
                           json.dumps(vars(done), indent=2) + "\n")
    return done


def main() -> None:
    args = parse_args()
    out = Path(args.output_dir)
    train_files, val_files = args.train_file, args.validation_file
    custom_files = train_files is not None or val_files is not None
    if args.dataset is not None and custom_files:
        raise ValueError("use either --dataset or custom source files, not both")
    if args.dataset is None and not custom_files:
        train_files, held_out = nanochat_climbmix_files(args.climbmix_train_shards)
        val_files = [held_out]
        print(f"source: NanoChat ClimbMix ({len(train_files)} train shards; "
              f"validation shard {CLIMBMIX_VALIDATION_SHARD:05d})")
    elif args.dataset is None and (train_files is None or val_files is None):
        raise ValueError("custom file staging requires both --train-file and --validation-file")

    tokenizer = None
    if args.tokenizer:
        tokenizer = get_tokenizer(hf_name=args.tokenizer, prefer_hf=True,
                                  local_files_only=args.tokenizer_local_files_only)
    plan = ((args.train_split, "train", args.train_documents, train_files),
            (args.validation_split, "validation", args.validation_documents, val_files))
    for source_split, name, limit, files in plan:
        staged = stage_split(dataset_name=args.dataset, dataset_config=args.dataset_config,
                             source_files=files, source_split=source_split, output_split=name,
                             text_column=args.text_column, max_documents=limit, output_dir=out,
                             force=args.force, skip_existing=args.skip_existing,
                             tokenizer=tokenizer, tokenizer_batch_size=args.tokenizer_batch_size)
        path = out / f"{name}.jsonl"
        if staged is None:
            print(f"reuse {name}: {path}")
            continue
        tokens = f", {staged.tokens:,} tokens" if staged.tokens is not None else ""
        print(f"staged {name}: {staged.documents:,} documents, "
              f"{staged.utf8_bytes / 2**20:.2f} MiB{tokens} -> {path}")


if __name__ == "__main__":
    main()
