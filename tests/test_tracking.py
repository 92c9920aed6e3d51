"""Experiment-tracker selection and adapters (reference suite: tests/test_tracking.py:71-260)."""

from __future__ import annotations

import json
import types

import pytest

from ohara_b200 import tracking
from ohara_b200.tracking import (
    JsonlLogger,
    NullLogger,
    TrackioLogger,
    WandbLogger,
    create_logger,
    wandb_is_configured,
)


class Recorder:
    """Stands in for a tracker module: records init / log / finish calls."""

    def __init__(self, fail_init: bool = False, fail_finish: bool = False) -> None:
        self.inits, self.logs, self.finished = [], [], 0
        self.fail_init, self.fail_finish = fail_init, fail_finish
        self.run = types.SimpleNamespace(logs=[], finished=0)
        self.run.log = lambda metrics, step=None: self.run.logs.append((metrics, step))
        self.run.finish = lambda: setattr(self.run, "finished", self.run.finished + 1)

    def init(self, **kwargs):
        if self.fail_init:
            raise RuntimeError("cannot start a run")
        self.inits.append(kwargs)
        return self.run

    def log(self, metrics, **kwargs):
        self.logs.append((metrics, kwargs))

    def finish(self):
        if self.fail_finish:
            raise RuntimeError("cannot close")
        self.finished += 1


@pytest.fixture()
def world(monkeypatch):
    """Control which tracker modules 'exist', what importing them returns, and wandb's login."""
    state = types.SimpleNamespace(modules={}, wandb_ready=False)
    monkeypatch.setattr(tracking, "_module_available", lambda name: name in state.modules)
    monkeypatch.setattr(tracking.importlib, "import_module", lambda name: state.modules[name])
    monkeypatch.setattr(tracking, "wandb_is_configured", lambda: state.wandb_ready)
    return state


def make(backend="auto", **kwargs):
    return create_logger(backend, project="p", run_name="r", config={"lr": 1}, verbose=False, **kwargs)


def test_auto_prefers_wandb_then_trackio_then_nothing(world):
    world.modules = {"wandb": Recorder(), "trackio": Recorder()}
    world.wandb_ready = True
    assert isinstance(make(), WandbLogger)
    world.wandb_ready = False
    assert isinstance(make(), TrackioLogger)
    world.modules = {"trackio": Recorder()}
    assert isinstance(make(), TrackioLogger)
    world.modules, world.wandb_ready = {"wandb": Recorder(fail_init=True), "trackio": Recorder()}, True
    assert isinstance(make(), TrackioLogger)
    world.modules = {"trackio": Recorder(fail_init=True)}
    assert isinstance(make(), NullLogger)
    world.modules = {}
    nothing = make()
    assert isinstance(nothing, NullLogger)
    nothing.log_metrics({"loss": 1.0}, step=3)
    nothing.finish()


def test_explicit_backends_fail_loudly(world):
    assert isinstance(make("none"), NullLogger)
    with pytest.raises(RuntimeError, match="not installed"):
        make("wandb")
    with pytest.raises(RuntimeError, match="not installed"):
        make("trackio")
    world.modules = {"wandb": Recorder()}
    with pytest.raises(RuntimeError, match="API key"):
        make("wandb")
    with pytest.raises(ValueError, match="backend must be one of"):
        make("tensorboard")


def test_wandb_adapter_forwards_calls(world):
    module = Recorder()
    world.modules, world.wandb_ready = {"wandb": module}, True
    logger = make("wandb")
    assert module.inits == [{"project": "p", "name": "r", "config": {"lr": 1}}]
    logger.log_metrics({"loss": 2.0}, step=5)
    logger.log_metrics({"loss": 1.0})
    assert module.logs == [({"loss": 2.0}, {"step": 5}), ({"loss": 1.0}, {})]
    logger.finish()
    assert module.finished == 1
    broken = WandbLogger(Recorder(fail_finish=True), project="p", run_name=None, config=None)
    broken.finish()  # a tracker that cannot close must not fail the run


def test_trackio_adapter_renames_and_deduplicates(world):
    module = Recorder()
    world.modules = {"trackio": module}
    logger = make("trackio")
    logger.log_metrics({"loss": 1.0, "time": 0.5, "step": 9}, step=1)
    logger.log_metrics({"loss": 1.0, "val_loss": 2.0}, step=1)
    logger.log_metrics({"loss": 0.9}, step=2)
    assert module.logs == [], "metrics go to the run returned by init, not the module"
    assert module.run.logs == [({"loss": 1.0, "step_time_s": 0.5, "logged_step": 9}, 1),
                               ({"val_loss": 2.0}, 1), ({"loss": 0.9}, 2)]
    logger.finish()
    logger.finish()
    assert module.run.finished == 1 and module.finished == 0


def test_jsonl_backend_and_engine_contract(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    logger = create_logger("jsonl", project="p", run_name="r", config={"lr": 1}, verbose=False)
    assert isinstance(logger, JsonlLogger)
    logger.log_metrics({"loss": 3.0}, step=1)
    logger.finish()
    records = [json.loads(line) for line in logger.path.read_text().splitlines()]
    assert records[0] == {"config": {"lr": 1}} and records[1]["loss"] == 3.0 and records[1]["step"] == 1

    from ohara_b200 import OharaEngine

    seen = []
    sink = types.SimpleNamespace(log_metrics=lambda payload, step=None: seen.append((dict(payload), step)),
                                 finish=lambda: None)
    engine = OharaEngine(loggers=[sink])
    engine.log_dict({"loss": 1.5}, step=4)
    assert seen == [({"loss": 1.5}, 4)]


def test_wandb_configuration_detection(monkeypatch):
    for name in ("WANDB_MODE", "WANDB_API_KEY"):
        monkeypatch.delenv(name, raising=False)
    monkeypatch.setenv("WANDB_API_KEY", "k")
    assert wandb_is_configured()
    monkeypatch.delenv("WANDB_API_KEY")
    for mode, expected in (("offline", True), ("dryrun", True), ("disabled", False)):
        monkeypatch.setenv("WANDB_MODE", mode)
        assert wandb_is_configured() is expected
    monkeypatch.delenv("WANDB_MODE")
    monkeypatch.setitem(__import__("sys").modules, "wandb",
                        types.SimpleNamespace(api=types.SimpleNamespace(api_key=None)))
    assert not wandb_is_configured()
    monkeypatch.setitem(__import__("sys").modules, "wandb", None)  # import raises ImportError
    assert not wandb_is_configured()
