"""Tracing and timing helpers: NVTX ranges, device-side section timers, roofline fractions.

The reference has no tracing at all: wall-clock around a synchronised step is its only timer
(ohara/trainer.py:410-411, 506-508). Three small pieces replace that here.

``nvtx_range(name)``
    A context manager (and decorator) that opens an NVTX range when ranges are switched on
    (``OHARA_NVTX=1`` or ``enable_nvtx(True)``) and a CUDA device is present; otherwise it is the
    same shared no-op object every time, so it can stay in hot paths. The fused compute +
    collective paths (sharded optimizer, tensor / context / expert parallelism) and the phases of a
    training step are bracketed with it, so a timeline tool shows them by name.

``nvtx_annotate(name)`` is the decorator form.

``DeviceTimer``
    Named sections timed with CUDA events on the current stream (``time.perf_counter`` without a
    CUDA device). Nothing synchronises while sections are recorded; ``summary()`` synchronises once,
    reduces every section with MAX over the ranks of a process group - the time of a step of a
    multi-GPU job is that of its slowest rank - and returns milliseconds per section.

``roofline(...)``
    Given the FLOPs and the bytes a kernel or step must move through HBM and over NVLink, the time
    each resource needs at the measured peaks (``MEASURED_PEAKS.json``: copy bandwidth and cuBLAS
    bf16 rate, or the documented fallback figures), the binding resource, and the fraction of that
    bound which a measured duration achieves.
"""

from __future__ import annotations

import json
import os
import time
import functools
from contextlib import ContextDecorator, contextmanager
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.distributed as dist

# Fallback peaks (an earlier measurement on B200: stream copy and cuBLAS bf16) used when no
# MEASURED_PEAKS.json is found; NVLink: measured peer copy per direction per GPU.
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NVLINK_GBS = 770.0

_nvtx_enabled = os.environ.get("OHARA_NVTX", "0") not in ("", "0", "false", "False")


def enable_nvtx(enabled: bool = True) -> None:
    """Switch NVTX ranges on or off for this process (the default comes from ``OHARA_NVTX``)."""
    global _nvtx_enabled
    _nvtx_enabled = bool(enabled)


def nvtx_enabled() -> bool:
    return _nvtx_enabled and torch.cuda.is_available()


class _NoRange(ContextDecorator):
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _NvtxRange(ContextDecorator):
    def __init__(self, name: str) -> None:
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False


_NO_RANGE = _NoRange()


def nvtx_range(name: str):
    """``with nvtx_range("zero.reduce_scatter"): ...`` - a named range when enabled, else a no-op."""
    return _NvtxRange(name) if nvtx_enabled() else _NO_RANGE


def nvtx_annotate(name: str):
    """Decorator form of :func:`nvtx_range`; whether ranges are on is looked up at every call."""

    def wrap(fn):
        @functools.wraps(fn)
        def inner(*args, **kwargs):
            if not nvtx_enabled():
                return fn(*args, **kwargs)
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()

        return inner

    return wrap


class DeviceTimer:
    """Accumulates device time per named section.

    >>> timer = DeviceTimer()
    >>> with timer.section("forward"):
    ...     pass
    >>> timer.summary()            # {"forward": {"ms": ..., "calls": 1}}
    """

    def __init__(self, device: torch.device | str | None = None, group=None) -> None:
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.group = group
        self._events: dict[str, list[tuple]] = {}
        self._host_ms: dict[str, float] = {}
        self._calls: dict[str, int] = {}

    @property
    def on_device(self) -> bool:
        return self.device.type == "cuda"

    @contextmanager
    def section(self, name: str):
        self._calls[name] = self._calls.get(name, 0) + 1
        with nvtx_range(name):
            if self.on_device:
                begin = torch.cuda.Event(enable_timing=True)
                end = torch.cuda.Event(enable_timing=True)
                begin.record()
                try:
                    yield
                finally:
                    end.record()
                    self._events.setdefault(name, []).append((begin, end))
            else:
                started = time.perf_counter()
                try:
                    yield
                finally:
                    elapsed = (time.perf_counter() - started) * 1e3
                    self._host_ms[name] = self._host_ms.get(name, 0.0) + elapsed

    def reset(self) -> None:
        self._events.clear()
        self._host_ms.clear()
        self._calls.clear()

    def local_ms(self) -> dict[str, float]:
        """Milliseconds per section on this rank (synchronises the device once)."""
        totals = dict(self._host_ms)
        if self._events:
            torch.cuda.synchronize(self.device)
            for name, pairs in self._events.items():
                totals[name] = totals.get(name, 0.0) + sum(b.elapsed_time(e) for b, e in pairs)
        return totals

    def summary(self, reduce: bool = True) -> dict[str, dict[str, float]]:
        """``{section: {"ms": max over ranks, "calls": n}}``. Every rank must have recorded the
        same sections when ``reduce`` is on and a process group exists."""
        totals = self.local_ms()
        names = sorted(totals)
        values = [totals[n] for n in names]
        if reduce and names and dist.is_available() and dist.is_initialized():
            backend = dist.get_backend(self.group)
            device = self.device if backend == "nccl" else torch.device("cpu")
            packed = torch.tensor(values, dtype=torch.float64, device=device)
            dist.all_reduce(packed, op=dist.ReduceOp.MAX, group=self.group)
            values = packed.tolist()
        return {n: {"ms": float(v), "calls": self._calls.get(n, 0)} for n, v in zip(names, values)}


@dataclass
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    nvlink_gbs: float
    source: str  # "measured" or "fallback"


def load_peaks(path: str | os.PathLike | None = None) -> Peaks:
    """Peaks from ``MEASURED_PEAKS.json`` (``path``, ``OHARA_MEASURED_PEAKS`` or the file next to
    the package), else the fallback figures."""
    candidates = []
    if path is not None:
        candidates.append(Path(path))
    if os.environ.get("OHARA_MEASURED_PEAKS"):
        candidates.append(Path(os.environ["OHARA_MEASURED_PEAKS"]))
    candidates.append(Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json")
    for candidate in candidates:
        try:
            data = json.loads(candidate.read_text())
            burst = float(data["bf16_tflops"])
            return Peaks(float(data["hbm_gbs"]), burst,
                         float(data.get("bf16_tflops_sustained") or burst), NVLINK_GBS, "measured")
        except (OSError, ValueError, KeyError, TypeError):
            continue
    return Peaks(FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, 1400.0, NVLINK_GBS, "fallback")


def roofline(ms: float, *, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0,
             sustained: bool = False, peaks: Peaks | None = None) -> dict[str, float | str]:
    """Roofline of one measured duration.

    ``flops``: useful floating-point operations; ``hbm_bytes``: algorithmic bytes read + written;
    ``nvlink_bytes``: bytes that must leave (or enter) this GPU, per direction. ``sustained``
    selects the cuBLAS rate measured over seconds under the power cap (for a kernel timed inside a
    long step) instead of the burst rate. Returns the time each resource needs, the bound (the
    slowest of them), ``fraction`` = bound time / measured time, and which peaks were used."""
    if ms <= 0:
        raise ValueError("duration must be positive")
    peaks = peaks or load_peaks()
    rate = peaks.bf16_tflops_sustained if sustained else peaks.bf16_tflops
    needs = {
        "compute": flops / (rate * 1e12) * 1e3,
        "hbm": hbm_bytes / (peaks.hbm_gbs * 1e9) * 1e3,
        "nvlink": nvlink_bytes / (peaks.nvlink_gbs * 1e9) * 1e3,
    }
    bound = max(needs, key=needs.get)
    return {
        "ms": ms, "compute_ms": needs["compute"], "hbm_ms": needs["hbm"],
        "nvlink_ms": needs["nvlink"], "bound": bound, "bound_ms": needs[bound],
        "fraction": needs[bound] / ms, "peaks": f"of {peaks.source}",
        "achieved_tflops": flops / (ms * 1e-3) / 1e12,
        "achieved_hbm_gbs": hbm_bytes / (ms * 1e-3) / 1e9,
        "achieved_nvlink_gbs": nvlink_bytes / (ms * 1e-3) / 1e9,
    }
