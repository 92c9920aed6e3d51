"""Failure detection is exercised entirely on the host: fake stores and clocks for the unit tests,
gloo ranks on CPU for the multi-process cases. No device is involved."""

from __future__ import annotations

import io
import os
import subprocess
import sys
import textwrap
import threading
import time
from pathlib import Path

import pytest
import torch

from ohara_b200.runtime import (
    CollectiveTimeout,
    EngineConfig,
    FaultToleranceConfig,
    Heartbeat,
    OharaEngine,
    PeerFailure,
    StepWatchdog,
)

ROOT = Path(__file__).resolve().parents[1]


class DictStore:
    """In-memory stand-in for a c10d store (``add`` is the only call the heartbeat needs)."""

    def __init__(self) -> None:
        self.values: dict[str, int] = {}
        self.lock = threading.Lock()
        self.dropped: set[str] = set()

    def add(self, key: str, amount: int) -> int:
        with self.lock:
            if amount and key in self.dropped:  # a message the test loses on purpose
                return self.values.get(key, 0)
            self.values[key] = self.values.get(key, 0) + amount
            return self.values[key]


class ManualClock:
    def __init__(self) -> None:
        self.now = 0.0

    def __call__(self) -> float:
        return self.now


def test_heartbeat_flags_a_silent_rank_and_recovers_when_it_speaks_again():
    store, clock = DictStore(), ManualClock()
    beats = [Heartbeat(store, r, 3, interval_s=1.0, timeout_s=5.0, clock=clock) for r in range(3)]
    for step in range(4):
        clock.now = float(step)
        for hb in beats:
            hb.beat()
        for hb in beats:
            hb.poll()
    beats[0].check()
    # rank 2's heartbeats are lost from now on
    store.dropped.add(beats[2]._beat_key(2))
    for step in range(4, 12):
        clock.now = float(step)
        for hb in beats:
            hb.beat()
        beats[0].poll()
    assert beats[0].failed_ranks == [2]
    with pytest.raises(PeerFailure) as info:
        beats[0].check()
    assert info.value.failed == [2] and "rank(s) [2]" in str(info.value)
    # the messages get through again: the rank is no longer reported
    store.dropped.clear()
    clock.now = 13.0
    beats[2].beat()
    beats[0].poll()
    beats[0].check()


def test_heartbeat_departure_is_seen_immediately():
    store, clock = DictStore(), ManualClock()
    a = Heartbeat(store, 0, 2, interval_s=1.0, timeout_s=5.0, clock=clock)
    b = Heartbeat(store, 1, 2, interval_s=1.0, timeout_s=5.0, clock=clock)
    a.beat(); b.beat(); a.poll()
    b.leave()
    with pytest.raises(PeerFailure) as info:
        a.check(refresh=True)
    assert info.value.left == [1] and info.value.failed == []
    assert a.departed_ranks == [1]


def test_heartbeat_thread_runs_and_stops():
    store = DictStore()
    with Heartbeat(store, 0, 2, interval_s=0.02, timeout_s=0.2) as hb:
        time.sleep(0.5)
        assert store.values[hb._beat_key(0)] > 3
        assert hb.failed_ranks == [1]  # rank 1 never said anything
    count = store.values[hb._beat_key(0)]
    time.sleep(0.1)
    assert store.values[hb._beat_key(0)] == count


def test_heartbeat_rejects_bad_timing():
    with pytest.raises(ValueError):
        Heartbeat(DictStore(), 0, 2, interval_s=2.0, timeout_s=1.0)


def test_step_watchdog_fires_only_for_a_late_step():
    fired: list[tuple[int, float]] = []
    stream = io.StringIO()
    dog = StepWatchdog(0.15, on_timeout=lambda step, elapsed: fired.append((step, elapsed)),
                       stream=stream, poll_s=0.02)
    try:
        with dog.step(1):
            time.sleep(0.02)
        time.sleep(0.25)
        assert fired == []
        with dog.step(2):
            time.sleep(0.4)
        assert [step for step, _ in fired] == [2] and fired[0][1] >= 0.15
        assert dog.expired_steps == [2]
        assert "step 2 exceeded" in stream.getvalue()
    finally:
        dog.close()


def test_collective_timeout_is_a_runtime_error():
    assert issubclass(CollectiveTimeout, RuntimeError)
    from ohara_b200 import ops

    assert ops.CollectiveTimeout is CollectiveTimeout


def test_engine_guard_is_a_no_op_without_configuration():
    engine = OharaEngine(EngineConfig())
    engine.launch()
    engine.check_peers()
    with engine.guard_step(1):
        pass
    engine.close()
    engine = OharaEngine(EngineConfig(fault_tolerance=FaultToleranceConfig(step_timeout_s=5.0)))
    engine.launch()
    assert engine.watchdog is not None
    with engine.guard_step(3):
        pass
    engine.close()
    assert engine.watchdog is None


def _run_ranks(script: str, world: int, tmp_path, timeout=180):
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(30100 + os.getpid() % 400), str(path)]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


def test_ranks_learn_on_the_host_that_a_peer_left_or_died(tmp_path):
    """Rank 2 announces its departure after step 2; rank 1 exits without a word after step 4. The
    survivors see both on the host, before they would issue the next collective."""
    proc = _run_ranks(
        """
        import os, sys, time
        import torch, torch.distributed as dist
        from ohara_b200.runtime import (EngineConfig, FaultToleranceConfig, OharaEngine,
                                        ParallelConfig, PeerFailure)
        engine = OharaEngine(EngineConfig(
            parallel=ParallelConfig(dp_replicate=3),
            fault_tolerance=FaultToleranceConfig(heartbeat_interval_s=0.1, heartbeat_timeout_s=1.0)))
        engine.launch()
        rank = engine.global_rank
        value = torch.ones(1)
        for step in range(1, 3):
            engine.check_peers()
            dist.all_reduce(value)
        assert value.item() == 9.0
        if rank == 2:
            engine.leave()          # between steps, nothing in flight
            os._exit(0)
        seen_left = seen_dead = False
        deadline = time.monotonic() + 20
        while time.monotonic() < deadline:
            try:
                engine.check_peers(refresh=True)
            except PeerFailure as failure:
                seen_left = failure.left == [2]
                break
            time.sleep(0.05)
        assert seen_left, "departure of rank 2 was not reported"
        if rank == 1:
            os._exit(0)             # dies silently
        deadline = time.monotonic() + 20
        while time.monotonic() < deadline:
            try:
                engine.check_peers(refresh=True)
            except PeerFailure as failure:
                if failure.failed == [1]:
                    seen_dead = True
                    break
            time.sleep(0.05)
        assert seen_dead, "silent death of rank 1 was not reported"
        print("SURVIVOR_OK", flush=True)
        os._exit(0)                 # peers are gone: skip the collective teardown
        """,
        3, tmp_path,
    )
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "SURVIVOR_OK" in proc.stdout


def test_short_process_group_timeout_ends_a_collective_with_an_error(tmp_path):
    """A rank never joins the collective: the others get an error after the short timeout
    instead of waiting forever. The absent rank stays alive until the waiting rank has reported,
    so the only thing that can end the wait is the timeout itself (not a closed connection)."""
    proc = _run_ranks(
        f"""
        import os, time
        from datetime import timedelta
        from pathlib import Path
        import torch, torch.distributed as dist
        done = Path({str(tmp_path / "reported")!r})
        dist.init_process_group("gloo", timeout=timedelta(seconds=3))
        rank = dist.get_rank()
        if rank == 1:
            deadline = time.monotonic() + 90
            while not done.exists() and time.monotonic() < deadline:
                time.sleep(0.1)     # alive, connected, but never joins
            os._exit(0)
        started = time.monotonic()
        try:
            dist.all_reduce(torch.ones(1))
        except Exception as error:
            waited = time.monotonic() - started
            print("TIMEOUT_OK", type(error).__name__, f"{{waited:.1f}}", flush=True)
            done.touch()
            os._exit(0 if waited < 60 else 4)
        done.touch()
        os._exit(3)
        """,
        2, tmp_path,
    )
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "TIMEOUT_OK" in proc.stdout


# -- a device-side timeout reaches the training loop ---------------------------------------------
class _FakeWorkspace:
    def __init__(self):
        self.aborted = 0

    def abort(self):
        self.aborted += 1


def test_engine_device_status_raises_and_releases_stream_waits(monkeypatch):
    """A status word that holds a timeout code makes ``check_device_status`` raise and, first,
    release the stream-ordered waits of every fused workspace of the prepared module."""
    import torch.nn as nn

    from ohara_b200 import ops
    from ohara_b200.errors import CollectiveTimeout

    engine = OharaEngine()
    engine.launch()
    engine.check_device_status()  # CPU: nothing to read, nothing raised

    class FakeExt:
        def status(self, clear):
            return [5, 17, 3, 0]  # "peer flag never written", block 17, three waits abandoned

    monkeypatch.setattr(ops, "ext", lambda: FakeExt())
    module = nn.Sequential(nn.Linear(2, 2), nn.Linear(2, 2))
    shared = _FakeWorkspace()
    module[0].workspace = shared
    module[1].workspace = shared          # one workspace shared by the layers: aborted once
    module[1].cp_workspace = _FakeWorkspace()
    engine._module = module
    engine._device = torch.device("cuda")  # pretend: only the type is looked at
    with pytest.raises(CollectiveTimeout, match="peer flag never written"):
        engine.check_device_status()
    assert shared.aborted == 1 and module[1].cp_workspace.aborted == 1
    engine._device = torch.device("cpu")
    engine.close()


def test_trainer_stops_and_does_not_checkpoint_after_a_device_timeout(tmp_path):
    """The step whose collective was abandoned must not be followed by another step, and must
    not be saved."""
    import torch.nn as nn
    from torch.utils.data import DataLoader, TensorDataset

    from ohara_b200.errors import CollectiveTimeout
    from ohara_b200.lr_scheduler import Scheduler
    from ohara_b200.trainer import Trainer

    class Engine(OharaEngine):
        checks = 0

        def check_device_status(self):
            self.checks += 1
            if self.checks == 2:
                raise CollectiveTimeout("ohara_b200 kernel wait timed out: peer flag never written")

    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(7, 7)

        def forward(self, x):
            return self.emb(x)

    engine = Engine()
    engine.launch()
    model = engine.prepare(Tiny())
    rows = torch.randint(0, 7, (16, 5))
    loader = DataLoader(TensorDataset(rows, rows), batch_size=4)
    path = tmp_path / "ckpt" / "model.pt"
    trainer = Trainer(engine, model, torch.optim.SGD(model.parameters(), lr=0.1), loader, loader,
                      Scheduler(0.1), micro_batch=1, max_iters=5, eval_iters=0, save_ckpt_iters=2,
                      checkpoint_path=path, print_every=10**9)
    with pytest.raises(CollectiveTimeout):
        trainer.train()
    assert engine.checks == 2            # raised after step 2, before its checkpoint
    assert not path.exists()
    assert trainer.train_batches_consumed == 2
    engine.close()


def test_workspace_abort_releases_its_own_flags_and_poisons_the_workspace(monkeypatch):
    """``abort()`` writes the release value into this rank's copies of the peers' "staged" flags
    (the words the copy streams wait on) and refuses further use."""
    from ohara_b200.parallel import cp, tp_fused

    calls = []
    for module in (tp_fused, cp):
        monkeypatch.setattr(module, "release_stream_waits",
                            lambda addresses, device=None: calls.append(list(addresses)))

    class Flags:
        pointers = [0x1000, 0x2000, 0x3000]

    tp = object.__new__(tp_fused.TPWorkspace)
    tp.world, tp.rank, tp.flags, tp.device, tp.poisoned = 3, 1, Flags(), None, False
    tp.abort()
    assert calls[-1] == [0x2000 + 4 * (tp_fused._AG_SLOT + r) for r in range(3)]
    with pytest.raises(RuntimeError, match="aborted"):
        tp.stage(torch.zeros(128, 8))
    ws = object.__new__(cp.CPWorkspace)
    ws.world, ws.rank, ws.flags, ws.device, ws.poisoned = 3, 2, Flags(), None, False
    ws.abort()
    assert calls[-1] == [0x3000 + 4 * (cp._KV_SLOT + r) for r in range(3)]
    with pytest.raises(RuntimeError, match="aborted"):
        ws.exchange_kv(torch.zeros(2, 1, 2, 1, 8))


def test_step_watchdog_expiry_releases_fused_waits():
    engine = OharaEngine(EngineConfig(fault_tolerance=FaultToleranceConfig(step_timeout_s=0.2)))
    engine.launch()
    released = []
    engine.abort_fused_waits = lambda: released.append(True) or 0
    with engine.guard_step(1):
        deadline = time.monotonic() + 5
        while not released and time.monotonic() < deadline:
            time.sleep(0.05)
    assert released
    engine.close()


def test_interrupted_save_keeps_the_previous_checkpoint_and_damaged_files_are_named(tmp_path, monkeypatch):
    """Host-side failure injection around checkpoints: a crash in the middle of a save leaves the
    last complete file in place and no temporary file behind; a truncated or foreign file raises
    ``CheckpointError`` with the path instead of loading garbage."""
    import torch

    from ohara_b200 import OharaEngine
    from ohara_b200.errors import CheckpointError

    engine = OharaEngine()
    path = tmp_path / "run" / "ckpt.pt"
    engine.save(path, {"idx": 1, "weights": torch.arange(4.0)})
    real_save = torch.save

    def dies_half_way(obj, file, *args, **kwargs):
        real_save(obj, file, *args, **kwargs)
        with open(file, "r+b") as handle:          # the temporary file is incomplete ...
            handle.truncate(10)
        raise OSError("disk full")                # ... when the process is interrupted

    monkeypatch.setattr(torch, "save", dies_half_way)
    with pytest.raises(OSError, match="disk full"):
        engine.save(path, {"idx": 2, "weights": torch.zeros(4)})
    monkeypatch.setattr(torch, "save", real_save)
    assert [p.name for p in path.parent.iterdir()] == ["ckpt.pt"]      # no temporary file left
    assert engine.load(path)["idx"] == 1                                 # the old one is intact

    whole = path.read_bytes()
    path.write_bytes(whole[: len(whole) // 2])
    with pytest.raises(CheckpointError, match="ckpt.pt"):
        engine.load(path)
    path.write_bytes(b"not a checkpoint at all")
    with pytest.raises(CheckpointError):
        engine.load(path)
    real_save([1, 2, 3], path)
    with pytest.raises(CheckpointError, match="list"):
        engine.load(path)
    with pytest.raises(FileNotFoundError):
        engine.load(tmp_path / "missing.pt")
