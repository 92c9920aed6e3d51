"""Human-readable random run names, e.g. ``quokka-2026_08_12_11_30_02``
(reference: ohara/utils/rand.py:1-22, which draws from a pokemon name list)."""

from __future__ import annotations

import random
from datetime import datetime
from functools import lru_cache
from pathlib import Path

_NAMES_FILE = Path(__file__).parent / "data" / "run_names.txt"


@lru_cache(maxsize=1)
def name_pool() -> tuple[str, ...]:
    return tuple(_NAMES_FILE.read_text(encoding="utf-8").split())


def random_name() -> str:
    stamp = datetime.now().strftime("%Y_%m_%d_%H_%M_%S")
    return f"{random.choice(name_pool())}-{stamp}"


def pokemon_names() -> tuple[str, ...]:
    """Name of this function in the reference (ohara/utils/rand.py:14); the pool here is this
    package's own list of run names."""
    return name_pool()
