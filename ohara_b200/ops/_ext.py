"""Loader for the in-tree sm_100a extension (``ohara_b200/_C*.so``).

The extension is built by ``python -m ohara_b200.build_ext`` (nvcc cross-compiles without a GPU).
``ext()`` imports it on first use and fails loudly when a CUDA device is present but the shared
object is missing or unloadable: a silent fallback to eager PyTorch on a GPU box would hide exactly
the code this package exists for.
"""

from __future__ import annotations

import importlib.util
import os
import sys
from types import ModuleType

_EXT: ModuleType | None = None
_ERROR: Exception | None = None


def _load() -> ModuleType:
    from ohara_b200 import build_ext

    path = build_ext.ext_path()
    if not path.exists():
        if os.environ.get("OHARA_B200_NO_JIT_BUILD"):
            raise ImportError(f"{path} is missing; run `python -m ohara_b200.build_ext`")
        build_ext.build()
    name = "ohara_b200._C"
    spec = importlib.util.spec_from_file_location(name, str(path))
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot load extension from {path}")
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def ext() -> ModuleType:
    """Return the compiled extension module, importing it on first call."""
    global _EXT, _ERROR
    if _EXT is not None:
        return _EXT
    if _ERROR is not None:
        raise RuntimeError("ohara_b200 CUDA extension failed to load earlier") from _ERROR
    try:
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        _EXT = _load()
    except Exception as error:  # pragma: no cover - exercised only on broken installs
        _ERROR = error
        raise RuntimeError(
            "the ohara_b200 CUDA extension is required on CUDA devices and could not be loaded: "
            f"{error}"
        ) from error
    return _EXT


def available() -> bool:
    """True when the extension can be imported (it may still need a GPU to run anything)."""
    try:
        ext()
        return True
    except RuntimeError:
        return False
