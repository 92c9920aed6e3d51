"""Hugging Face cache helpers (reference: ohara/utils/load.py:1-28)."""

from __future__ import annotations

import os

HF_CACHE_DIR = os.path.expanduser("~/.cache/huggingface/hub/")


def get_model_path(model_name: str) -> tuple[str | None, str | None]:
    """Locate a downloaded snapshot; returns ``(path, error)`` with exactly one ``None``."""
    snapshots = os.path.join(HF_CACHE_DIR, "models--" + model_name.replace("/", "--"), "snapshots")
    if not os.path.isdir(snapshots):
        return None, f"{model_name} is not in the local Hugging Face cache"
    revisions = sorted(os.listdir(snapshots))
    if not revisions:
        return None, f"{model_name} has no snapshot revisions on disk"
    return os.path.join(snapshots, revisions[0]), None


def download_hf_model(model_name: str) -> str:
    from huggingface_hub import snapshot_download

    return snapshot_download(model_name)
