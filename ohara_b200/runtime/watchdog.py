"""Host-side failure detection: peer heartbeats over the rendezvous store and a step watchdog.

The reference has no failure detector beyond the process-group timeout
(ohara/runtime/config.py:12, ohara/runtime/engine.py:144-147): a rank that died is noticed when the
next collective times out, half an hour later. Fused peer-memory collectives make that worse in
principle, because a kernel waiting on a flag of a dead rank can only give up after its own bounded
wait. Two host-side pieces close the gap; neither touches the device:

``Heartbeat``
    Every rank bumps a counter in the c10d key-value store from a daemon thread and watches the
    counters of its peers. A counter that stops moving for ``timeout_s`` marks that rank as failed;
    a rank that stops on purpose announces it (``leave``) so the others learn of it at once.
    ``check()`` is called on the host before a step is launched and raises ``PeerFailure`` instead
    of launching kernels that would wait on the missing rank.

``StepWatchdog``
    A deadline per step. If the step body does not finish in time the watchdog dumps the Python
    stacks, calls ``on_timeout`` and (optionally) ends the process with a distinctive exit code so
    that an elastic launcher can restart the job from its last checkpoint.

``CollectiveTimeout`` is the exception type raised when a device-side bounded wait ran out
(``ops.check_status``) or a c10d collective timed out.
"""

from __future__ import annotations

import faulthandler
import os
import sys
import threading
import time
from contextlib import contextmanager
from typing import Callable, Iterable

import torch.distributed as dist

from ohara_b200.errors import CollectiveTimeout  # noqa: F401  (re-exported)


class PeerFailure(RuntimeError):
    """One or more ranks stopped sending heartbeats or announced that they left."""

    def __init__(self, failed: Iterable[int], left: Iterable[int] = ()) -> None:
        self.failed = sorted(failed)
        self.left = sorted(left)
        parts = []
        if self.failed:
            parts.append(f"no heartbeat from rank(s) {self.failed}")
        if self.left:
            parts.append(f"rank(s) {self.left} left the job")
        super().__init__("; ".join(parts) or "peer failure")


WATCHDOG_EXIT_CODE = 75  # EX_TEMPFAIL: "try again later", what a restarting launcher wants to see


def default_store():
    """The store the default process group was created with (``None`` outside a job)."""
    if not dist.is_available() or not dist.is_initialized():
        return None
    from torch.distributed import distributed_c10d

    return distributed_c10d._get_default_store()


class Heartbeat:
    """Liveness of the ranks of a job through counters in a c10d store.

    ``store`` needs ``add(key, n) -> int`` and ``set(key, value)`` / ``get(key)`` (the c10d store
    interface); ``add(key, 0)`` is used as a non-blocking read. The store must outlive the ranks
    (under ``torchrun`` it lives in the agent process).
    """

    def __init__(self, store, rank: int, world_size: int, *, interval_s: float = 1.0,
                 timeout_s: float = 10.0, prefix: str = "ohara_b200/heartbeat",
                 clock: Callable[[], float] = time.monotonic) -> None:
        if interval_s <= 0 or timeout_s <= interval_s:
            raise ValueError("need 0 < interval_s < timeout_s")
        self.store = store
        self.rank = int(rank)
        self.world_size = int(world_size)
        self.interval_s = float(interval_s)
        self.timeout_s = float(timeout_s)
        self.prefix = prefix
        self._clock = clock
        self._lock = threading.Lock()
        self._last_value = {r: 0 for r in range(self.world_size) if r != self.rank}
        self._last_change = {r: clock() for r in self._last_value}
        self._failed: set[int] = set()
        self._left: set[int] = set()
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    # -- keys ------------------------------------------------------------------------------------
    def _beat_key(self, rank: int) -> str:
        return f"{self.prefix}/beat/{rank}"

    def _left_key(self, rank: int) -> str:
        return f"{self.prefix}/left/{rank}"

    # -- one tick (public for tests that drive the clock by hand) ----------------------------------
    def beat(self) -> None:
        self.store.add(self._beat_key(self.rank), 1)

    def poll(self) -> None:
        """Read every peer's counter once and update the failed / left sets."""
        now = self._clock()
        for peer in list(self._last_value):
            value = int(self.store.add(self._beat_key(peer), 0))
            gone = int(self.store.add(self._left_key(peer), 0)) > 0
            with self._lock:
                if gone:
                    self._left.add(peer)
                    self._failed.discard(peer)
                    continue
                if value != self._last_value[peer]:
                    self._last_value[peer] = value
                    self._last_change[peer] = now
                    self._failed.discard(peer)
                elif now - self._last_change[peer] > self.timeout_s:
                    self._failed.add(peer)

    # -- thread ----------------------------------------------------------------------------------
    def start(self) -> "Heartbeat":
        if self._thread is not None:
            return self
        self.beat()

        def run() -> None:
            while not self._stop.wait(self.interval_s):
                try:
                    self.beat()
                    self.poll()
                except Exception:  # the store went away: the launcher is tearing the job down
                    return

        self._thread = threading.Thread(target=run, name="ohara-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval_s * 4)
            self._thread = None

    def leave(self) -> None:
        """Announce a deliberate departure (call between steps, with nothing in flight)."""
        self.store.add(self._left_key(self.rank), 1)
        self.stop()

    # -- queries ---------------------------------------------------------------------------------
    @property
    def failed_ranks(self) -> list[int]:
        with self._lock:
            return sorted(self._failed)

    @property
    def departed_ranks(self) -> list[int]:
        with self._lock:
            return sorted(self._left)

    def check(self, *, refresh: bool = False) -> None:
        """Raise ``PeerFailure`` if a peer is known to be gone. ``refresh`` polls the store first
        (one round trip per peer) instead of relying on the background thread's last look."""
        if refresh:
            self.poll()
        with self._lock:
            if self._failed or self._left:
                raise PeerFailure(self._failed, self._left)

    def __enter__(self) -> "Heartbeat":
        return self.start()

    def __exit__(self, *exc) -> None:
        self.stop()


class StepWatchdog:
    """Deadline for the body of a training or serving step.

    ``with watchdog.step(index): ...`` arms the deadline; leaving the block disarms it. When the
    deadline passes, the watchdog thread writes all Python stacks to ``stream``, calls
    ``on_timeout(index, elapsed_s)`` and, with ``hard_exit=True``, ends the process with
    ``WATCHDOG_EXIT_CODE`` (a step that is stuck inside a driver call cannot be interrupted from
    Python; ending the process is what frees its peers, whose heartbeats then report it).
    """

    def __init__(self, timeout_s: float, *, on_timeout: Callable[[int, float], None] | None = None,
                 hard_exit: bool = False, stream=None, poll_s: float | None = None) -> None:
        if timeout_s <= 0:
            raise ValueError("timeout_s must be positive")
        self.timeout_s = float(timeout_s)
        self.on_timeout = on_timeout
        self.hard_exit = hard_exit
        self.stream = stream
        self.poll_s = poll_s if poll_s is not None else min(1.0, self.timeout_s / 4)
        self.expired_steps: list[int] = []
        self._lock = threading.Lock()
        self._armed_at: float | None = None
        self._step = -1
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="ohara-step-watchdog", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            with self._lock:
                armed_at, step = self._armed_at, self._step
            if armed_at is None:
                continue
            elapsed = time.monotonic() - armed_at
            if elapsed < self.timeout_s:
                continue
            with self._lock:
                if self._armed_at != armed_at:
                    continue  # the step finished while we were looking
                self._armed_at = None
                self.expired_steps.append(step)
            stream = self.stream if self.stream is not None else sys.stderr
            try:
                print(f"[watchdog] step {step} exceeded {self.timeout_s:.1f}s "
                      f"({elapsed:.1f}s); Python stacks follow", file=stream, flush=True)
                faulthandler.dump_traceback(file=stream, all_threads=True)
            except Exception:
                pass
            if self.on_timeout is not None:
                self.on_timeout(step, elapsed)
            if self.hard_exit:
                os._exit(WATCHDOG_EXIT_CODE)

    @contextmanager
    def step(self, index: int):
        with self._lock:
            self._step = int(index)
            self._armed_at = time.monotonic()
        try:
            yield self
        finally:
            with self._lock:
                self._armed_at = None

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=self.poll_s * 4)
