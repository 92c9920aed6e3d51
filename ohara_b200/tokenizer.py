"""Tokenizer loading with an explicit source priority, and the token → UTF-8 byte-length table
used for bits-per-byte evaluation (reference: ohara/tokenizer.py:21-211).

``transformers`` is imported lazily so that modules which only need the byte table or the result
type do not pay for it.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

LOCAL_TOKENIZER_FILES = (
    "tokenizer.json",
    "tokenizer_config.json",
    "special_tokens_map.json",
    "vocab.json",
    "merges.txt",
)


@dataclass
class TokenizerLoadResult:
    tokenizer: Any
    source: str  # "hf", "local" or "fallback_hf"
    identifier: str


def _has_local_tokenizer(path: Path) -> bool:
    return path.is_dir() and any((path / name).exists() for name in LOCAL_TOKENIZER_FILES)


def _load_hf_tokenizer(identifier: str, *, use_fast: bool = True, local_files_only: bool = False,
                       cache_dir: str | Path | None = None, **kwargs: Any):
    from transformers import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(
        identifier, use_fast=use_fast, local_files_only=local_files_only, cache_dir=cache_dir,
        **kwargs,
    )
    if tokenizer.pad_token_id is None and tokenizer.eos_token is not None:
        tokenizer.pad_token = tokenizer.eos_token
    if tokenizer.padding_side is None:
        tokenizer.padding_side = "right"
    return tokenizer


def load_tokenizer(*, hf_name: str | None = None, tokenizer_dir: str | Path = "./tokenizer",
                   prefer_hf: bool = True, fallback_hf_name: str | None = None,
                   use_fast: bool = True, local_files_only: bool = False,
                   cache_dir: str | Path | None = None, **kwargs: Any) -> TokenizerLoadResult:
    """Try sources in order and return the first that loads.

    ``prefer_hf=True``: hub name → local directory → fallback hub name;
    ``prefer_hf=False``: local directory → hub name → fallback hub name.
    """
    local_dir = Path(tokenizer_dir)
    local = [("local", str(local_dir), True)] if _has_local_tokenizer(local_dir) else []
    hub = [("hf", hf_name, False)] if hf_name else []
    attempts = (hub + local) if prefer_hf else (local + hub)
    if fallback_hf_name and fallback_hf_name != hf_name:
        attempts.append(("fallback_hf", fallback_hf_name, False))
    if not attempts:
        raise RuntimeError(
            "No tokenizer source configured. Pass `hf_name` or provide local tokenizer files in "
            f"`{local_dir}`."
        )
    errors = []
    for source, identifier, local_only in attempts:
        try:
            tokenizer = _load_hf_tokenizer(
                identifier, use_fast=use_fast, local_files_only=local_only or local_files_only,
                cache_dir=cache_dir, **kwargs,
            )
            return TokenizerLoadResult(tokenizer, source, identifier)
        except Exception as error:  # noqa: BLE001 - every failure is reported together below
            errors.append(f"{source}({identifier}): {type(error).__name__}: {error}")
    raise RuntimeError("Failed to load tokenizer. " + " | ".join(errors))


def get_tokenizer(**kwargs: Any):
    """``load_tokenizer(...).tokenizer``."""
    return load_tokenizer(**kwargs).tokenizer


def _read_token_bytes_cache(cache_file: Path, tokenizer, include_special: bool) -> torch.Tensor:
    with open(cache_file, "rb") as handle:
        payload = torch.load(handle, map_location="cpu", weights_only=True)
    if isinstance(payload, torch.Tensor):  # legacy tensor-only cache
        table = payload
    elif isinstance(payload, dict):
        table = payload.get("token_bytes")
        if not isinstance(table, torch.Tensor):
            raise ValueError(f"invalid token-byte cache: {cache_file}")
        if payload.get("tokenizer") != str(getattr(tokenizer, "name_or_path", "unknown")):
            raise ValueError(f"token-byte cache tokenizer mismatch: {cache_file}")
        if bool(payload.get("include_special")) != include_special:
            raise ValueError(f"token-byte cache special-token mode mismatch: {cache_file}")
    else:
        raise ValueError(f"invalid token-byte cache: {cache_file}")
    if table.ndim != 1 or table.numel() != len(tokenizer):
        raise ValueError(f"token-byte cache vocabulary mismatch: {cache_file}")
    return table


def get_token_bytes(tokenizer, *, device: str | torch.device = "cpu",
                    cache_path: str | Path | None = None,
                    include_special: bool = False) -> torch.Tensor:
    """int32 tensor mapping token id → number of UTF-8 bytes it decodes to. Special tokens count
    as zero bytes unless ``include_special``. With ``cache_path`` the table is stored atomically
    and validated against the tokenizer on reload."""
    cache_file = Path(cache_path) if cache_path is not None else None
    if cache_file is not None and cache_file.exists():
        return _read_token_bytes_cache(cache_file, tokenizer, include_special).to(device=device)
    size = len(tokenizer)
    skip = set() if include_special else set(getattr(tokenizer, "all_special_ids", []) or [])
    table = torch.zeros(size, dtype=torch.int32)
    for token_id in range(size):
        if token_id in skip:
            continue
        table[token_id] = len(tokenizer.decode([token_id], skip_special_tokens=False).encode("utf-8"))
    if cache_file is not None:
        cache_file.parent.mkdir(parents=True, exist_ok=True)
        temporary = cache_file.with_name(f".{cache_file.name}.tmp-{os.getpid()}")
        try:
            with open(temporary, "wb") as handle:
                torch.save({"tokenizer": str(getattr(tokenizer, "name_or_path", "unknown")),
                            "include_special": include_special, "token_bytes": table}, handle)
            os.replace(temporary, cache_file)
        finally:
            temporary.unlink(missing_ok=True)
    return table.to(device=device)


def tokenizer_info(tokenizer) -> dict[str, Any]:
    return {
        "name_or_path": getattr(tokenizer, "name_or_path", "unknown"),
        "vocab_size": len(tokenizer),
        "pad_token_id": tokenizer.pad_token_id,
        "eos_token_id": tokenizer.eos_token_id,
        "bos_token_id": tokenizer.bos_token_id,
        "special_tokens": list(getattr(tokenizer, "all_special_tokens", []) or []),
    }


def __getattr__(name: str):
    """``AutoTokenizer`` is reachable as an attribute of this module, as in the reference (where
    it is imported at the top: ohara/tokenizer.py), without importing ``transformers`` until it
    is asked for."""
    if name == "AutoTokenizer":
        from transformers import AutoTokenizer

        return AutoTokenizer
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
