"""Tokenise a staged corpus once into flat ``uint16`` token bins.

    python examples/pretokenize_corpus.py --corpus ./data/scaling_corpus

Reads ``{split}.jsonl`` (as written by prepare_scaling_data.py) and writes ``{split}.bin`` plus a
JSON sidecar beside it. Training memory-maps the bins instead of tokenising inside the loop, which
is what otherwise keeps the GPUs waiting. Run once per (corpus, tokenizer) pair: the sidecar
records the vocabulary, so a mismatch fails at load instead of training on garbage ids.
Flags follow the reference entry point (examples/pretokenize_corpus.py:28-43).
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path
from typing import Iterator

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

from ohara_b200.chat import add_chat_tokens
from ohara_b200.tokenbin import read_token_bin_metadata, write_token_bin
from ohara_b200.tokenizer import get_tokenizer


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Pre-tokenise a staged corpus into token bins")
    p.add_argument("--corpus", default="./data/scaling_corpus")
    p.add_argument("--splits", default="train,validation")
    p.add_argument("--tokenizer", default="EleutherAI/gpt-neo-125m")
    p.add_argument("--tokenizer-local-files-only", action="store_true")
    p.add_argument("--chat-tokens", action="store_true",
                   help="reserve the chat special tokens, matching --chat-tokens at train time")
    p.add_argument("--text-column", default="text")
    p.add_argument("--batch-size", type=int, default=1024)
    p.add_argument("--force", action="store_true")
    return p.parse_args()


def read_jsonl(path: Path, text_column: str) -> Iterator[str]:
    with open(path, encoding="utf-8") as handle:
        for line in handle:
            if not line.strip():
                continue
            text = json.loads(line).get(text_column)
            if isinstance(text, str) and text:
                yield text


def main() -> None:
    args = parse_args()
    corpus = Path(args.corpus)
    if not corpus.is_dir():
        raise NotADirectoryError(f"corpus directory not found: {corpus}")
    tokenizer = get_tokenizer(hf_name=args.tokenizer, prefer_hf=True,
                              local_files_only=args.tokenizer_local_files_only)
    if args.chat_tokens:
        add_chat_tokens(tokenizer)
    print(f"tokenizer {args.tokenizer}: vocab {len(tokenizer):,}")

    for split in filter(None, (s.strip() for s in args.splits.split(","))):
        source, target = corpus / f"{split}.jsonl", corpus / f"{split}.bin"
        if not source.exists():
            raise FileNotFoundError(f"missing staged split: {source}")
        if target.exists() and not args.force:
            existing = read_token_bin_metadata(target)
            if existing["vocab_size"] != len(tokenizer):
                raise FileExistsError(
                    f"{target} was built with a {existing['vocab_size']:,} token vocabulary but "
                    f"this run has {len(tokenizer):,}; pass --force to rebuild")
            print(f"reuse {target}: {existing['tokens']:,} tokens")
            continue
        print(f"tokenizing {source} -> {target}")
        started = time.perf_counter()
        meta = write_token_bin(read_jsonl(source, args.text_column), tokenizer, target,
                               batch_size=args.batch_size)
        elapsed = time.perf_counter() - started
        print(f"  {meta['tokens']:,} tokens in {elapsed / 60:.1f}m "
              f"({meta['tokens'] / max(elapsed, 1e-9) / 1e6:.2f}M tokens/s), "
              f"{target.stat().st_size / 1e9:.2f} GB")


if __name__ == "__main__":
    main()
