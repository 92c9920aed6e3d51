"""Shared test doubles. Nothing here touches the network or a GPU."""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ohara_b200.chat import add_chat_tokens
from ohara_b200.models.llama import Config, Llama


class WordTokenizer:
    """A tiny closed-vocabulary tokenizer exposing the slice of the Hugging Face interface that
    the framework uses: lower-case letters, digits, space and a little punctuation are one token
    each; ``<doc>`` is BOS, EOS and PAD at once; special tokens can be added later and are matched
    greedily while encoding."""

    ALPHABET = "abcdefghijklmnopqrstuvwxyz0123456789 .,:?!\n-()+=*/"

    def __init__(self, name: str = "word-tokenizer") -> None:
        self.name_or_path = name
        self._tokens = ["<doc>"] + list(self.ALPHABET)
        self._index = {token: i for i, token in enumerate(self._tokens)}
        self._specials = ["<doc>"]
        self.bos_token_id = self.eos_token_id = self.pad_token_id = 0
        self.padding_side = "right"

    # -- vocabulary ------------------------------------------------------------------------------
    def __len__(self) -> int:
        return len(self._tokens)

    @property
    def vocab_size(self) -> int:
        return len(self._tokens)

    def get_vocab(self) -> dict[str, int]:
        return dict(self._index)

    @property
    def all_special_ids(self) -> list[int]:
        return [self._index[token] for token in self._specials]

    @property
    def all_special_tokens(self) -> list[str]:
        return list(self._specials)

    def add_special_tokens(self, mapping) -> int:
        added = 0
        for token in mapping["additional_special_tokens"]:
            if token not in self._index:
                self._index[token] = len(self._tokens)
                self._tokens.append(token)
                self._specials.append(token)
                added += 1
        return added

    def convert_tokens_to_ids(self, token: str):
        return self._index.get(token)

    # -- text <-> ids ----------------------------------------------------------------------------
    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids, position = [], 0
        multi = sorted((t for t in self._specials), key=len, reverse=True)
        while position < len(text):
            for token in multi:
                if text.startswith(token, position):
                    ids.append(self._index[token])
                    position += len(token)
                    break
            else:
                char = text[position].lower()
                if char in self._index:
                    ids.append(self._index[char])
                position += 1
        return ids

    def __call__(self, texts, add_special_tokens: bool = False, **_):
        if isinstance(texts, str):
            return {"input_ids": self.encode(texts)}
        return {"input_ids": [self.encode(text) for text in texts]}

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        pieces = []
        for token_id in ids:
            token = self._tokens[int(token_id)] if 0 <= int(token_id) < len(self._tokens) else ""
            if skip_special_tokens and token in self._specials:
                continue
            pieces.append(token)
        return "".join(pieces)

    def save_pretrained(self, directory) -> None:
        directory = Path(directory)
        directory.mkdir(parents=True, exist_ok=True)
        (directory / "tokenizer.json").write_text(json.dumps({"tokens": self._tokens}))


def chat_tokenizer() -> WordTokenizer:
    tokenizer = WordTokenizer()
    add_chat_tokens(tokenizer)
    return tokenizer


def tiny_llama(vocab_size: int, *, context: int = 64, seed: int = 0, **overrides) -> Llama:
    torch.manual_seed(seed)
    settings = dict(vocab_size=vocab_size, hidden_size=32, intermediate_size=64,
                    max_sequence_length=context, num_hidden_layers=2, num_attention_heads=2,
                    dropout=0.0)
    settings.update(overrides)
    return Llama(Config(**settings))


def exchange(question: str, answer) -> dict:
    return {"messages": [{"role": "user", "content": question},
                         {"role": "assistant", "content": answer}]}


def run_ranks(script, world: int, *, port: int, env: dict | None = None, timeout: float = 400.0,
              args: tuple = ()):
    """Run ``script`` as ``world`` processes with the rendezvous variables ``torchrun`` would set
    (RANK, LOCAL_RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT), without the launcher process in
    between. Returns ``(returncode, stdout, stderr)`` with the outputs of all ranks joined; if a
    rank fails or the time runs out, the ranks still running are stopped (by their own PIDs)."""
    import os
    import subprocess
    import sys
    import tempfile
    import time

    base = dict(os.environ if env is None else env)
    base.update(WORLD_SIZE=str(world), LOCAL_WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                MASTER_PORT=str(port))
    logs, procs = [], []
    for rank in range(world):
        out = tempfile.TemporaryFile(mode="w+")
        err = tempfile.TemporaryFile(mode="w+")
        logs.append((out, err))
        procs.append(subprocess.Popen(
            [sys.executable, str(script), *map(str, args)], stdout=out, stderr=err,
            env=dict(base, RANK=str(rank), LOCAL_RANK=str(rank), GROUP_RANK="0")))
    deadline = time.monotonic() + timeout
    code = 0
    while True:
        states = [proc.poll() for proc in procs]
        failed = [state for state in states if state not in (None, 0)]
        if failed:
            code = failed[0]
            break
        if all(state == 0 for state in states):
            break
        if time.monotonic() > deadline:
            code = -9
            break
        time.sleep(0.05)
    for proc in procs:
        if proc.poll() is None:
            proc.kill()
        proc.wait()
    stdout, stderr = [], []
    for out, err in logs:
        for handle, sink in ((out, stdout), (err, stderr)):
            handle.seek(0)
            sink.append(handle.read())
            handle.close()
    return code, "".join(stdout), "".join(stderr)


def launch_ranks(script, world: int, *, port: int, env: dict | None = None, timeout: float = 400.0,
                 args: tuple = ()):
    """:func:`run_ranks` with the result shaped like ``subprocess.CompletedProcess``."""
    import subprocess

    code, stdout, stderr = run_ranks(script, world, port=port, env=env, timeout=timeout, args=args)
    return subprocess.CompletedProcess([str(script), *map(str, args)], code, stdout, stderr)
