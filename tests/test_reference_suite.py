"""Runs the reference project's own test suite against this package (``import ohara`` is aliased
to ``ohara_b200``) when ``OHARA_REFERENCE_TESTS`` names the reference's ``tests`` folder. The
suite is not vendored, so without the variable the test is skipped."""

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SUITE = os.environ.get("OHARA_REFERENCE_TESTS")


@pytest.mark.skipif(not SUITE or not Path(SUITE).is_dir(),
                    reason="OHARA_REFERENCE_TESTS does not point at the reference's tests folder")
def test_the_reference_suite_passes_against_this_package():
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1",
               PYTHONPATH=os.pathsep.join([str(ROOT / "tests" / "reference_suite"), str(ROOT)]))
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", "-p", "ohara_alias", "-p", "no:cacheprovider", SUITE, "-q"],
        env=env, capture_output=True, text=True, timeout=1800, cwd=ROOT)
    tail = proc.stdout[-3000:]
    assert proc.returncode == 0, tail
    passed = int(re.search(r"(\d+) passed", tail).group(1))
    assert passed >= 200, tail


def _load(path: Path, name: str):
    import importlib.util

    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


@pytest.mark.skipif(not SUITE or not (Path(SUITE).parent / "experiments").is_dir(),
                    reason="no reference experiments folder beside OHARA_REFERENCE_TESTS")
def test_experiment_modules_compute_what_the_reference_files_compute():
    """The stand-alone pieces of ``experiments/`` whose counterparts in the reference import
    cleanly: same weights (or inputs) in, same numbers out."""
    import types

    import torch

    theirs, ours = Path(SUITE).parent / "experiments", ROOT / "experiments"
    package_alias = str(ROOT / "tests" / "reference_suite")
    sys.path[:0] = [package_alias, str(ROOT)]
    try:
        import ohara_alias  # noqa: F401  (their files import ``ohara``: give them this package)
    except ImportError:
        pass
    stubs = []
    for missing in ("lightning", "wandb", "datasets"):
        if missing not in sys.modules:
            try:
                __import__(missing)
            except Exception:  # noqa: BLE001 - any failure means "stub it"
                sys.modules[missing] = types.ModuleType(missing)
                stubs.append(missing)
    try:
        _compare_experiment_modules(theirs, ours)
    finally:  # leave no alias behind for tests that import the real reference package
        sys.meta_path[:] = [finder for finder in sys.meta_path
                            if type(finder).__module__ != "ohara_alias"]
        for name in [n for n in sys.modules if n == "ohara" or n.startswith("ohara.")] + stubs:
            sys.modules.pop(name, None)


def _compare_experiment_modules(theirs: Path, ours: Path) -> None:
    import torch

    torch.manual_seed(0)
    x = torch.randn(3, 7, 16)

    a, b = _load(theirs / "q_sparse/q_sparse.py", "ref_q_sparse"), _load(ours / "q_sparse/q_sparse.py", "our_q_sparse")
    left, right = x.clone().requires_grad_(), x.clone().requires_grad_()
    out_a, out_b = a.q_sparse(left, 5), b.q_sparse(right, 5)
    out_a.sum().backward(), out_b.sum().backward()
    assert torch.equal(out_a, out_b) and torch.equal(left.grad, right.grad)
    layer_a, layer_b = a.QSparseLinear(0.4, 16, 8), b.QSparseLinear(0.4, 16, 8)
    layer_b.load_state_dict(layer_a.state_dict())
    assert torch.equal(layer_a(x), layer_b(x))

    a, b = _load(theirs / "xglu/xglu.py", "ref_xglu"), _load(ours / "xglu/xglu.py", "our_xglu")
    layer_a, layer_b = a.XGLU(16, 32, xglu_rank=4), b.XGLU(16, 32, xglu_rank=4)
    layer_b.load_state_dict(layer_a.state_dict())
    torch.testing.assert_close(layer_a(x), layer_b(x))

    a = _load(theirs / "tokenformer/pattention.py", "ref_pattention")
    b = _load(ours / "misc/small_modules.py", "our_small_modules")
    torch.testing.assert_close(a.gelu_l2_norm(x), b.gelu_l2_norm(x))
    layer_a, layer_b = a.Pattention(16, 8, 10), b.Pattention(16, 8, 10)
    with torch.no_grad():
        layer_b.keys.copy_(layer_a.key_param_tokens)
        layer_b.values.copy_(layer_a.value_param_tokens)
    torch.testing.assert_close(layer_a(x), layer_b(x))

    hs = _load(theirs / "hypersphere/hs.py", "ref_hypersphere")
    layer_a, layer_b = hs.XLinear(16, 8), b.XLinear(16, 8)
    layer_b.load_state_dict(layer_a.state_dict())
    torch.testing.assert_close(layer_a(x), layer_b(x))

    galore = _load(theirs / "galore/galore.py", "ref_galore")
    for gradient in (torch.randn(12, 3) @ torch.randn(3, 20), torch.randn(30, 8)):
        low_a = galore.GaLoreProjector(rank=3).project(gradient, 0)
        low_b = b.GaLoreProjector(rank=3).project(gradient, 0)
        torch.testing.assert_close(low_a, low_b)

    a, b = _load(theirs / "mihawk/state_shift.py", "ref_shift"), _load(ours / "mihawk/state_shift.py", "our_shift")
    states = torch.randn(2, 9, 4)
    assert torch.equal(a.states_shift(states, 2), b.states_shift(states, 2))
    torch.testing.assert_close(a.state_predition_loss(states, 2), b.state_prediction_loss(states, 2))

    sys.path.insert(0, str(theirs / "mHC"))              # their model imports ``sinkhorn`` beside it
    try:
        a = _load(theirs / "mHC/model.py", "ref_mhc_model")
    finally:
        sys.path.remove(str(theirs / "mHC"))
    b = _load(ours / "mhc/hyper_connections.py", "our_hyper_connections")
    layer_a, layer_b = (m.ManifoldHyperConnections(16, 3, sinkhorn_iters=5) for m in (a, b))
    with torch.no_grad():
        for parameter in layer_a.parameters():
            parameter.add_(torch.randn_like(parameter) * 0.3)
    layer_b.load_state_dict(layer_a.state_dict())
    streams = torch.randn(2, 5, 3, 16)
    for got, want in zip(layer_b(streams), layer_a(streams)):
        torch.testing.assert_close(got, want)

    a, b = _load(theirs / "deepseek_moe/dsmoe.py", "ref_dsmoe"), _load(ours / "deepseek_moe/dsmoe.py", "our_dsmoe")
    settings = dict(num_experts=4, experts_per_token=2, num_shared_experts=1, aux_free_loadbalancing=True)
    layer_a, layer_b = a.DSMoE(16, 32, dropout=0.0, **settings), b.DSMoE(16, 32, **settings)
    layer_b.load_state_dict(layer_a.state_dict())
    # With all biases at zero the layers agree exactly, and the first update moves the biases the
    # same way. Later outputs may differ on purpose: once a bias changes which experts are picked,
    # the reference still weights them with the largest unbiased scores in order, whatever was
    # picked (dsmoe.py:181), this package with the scores of the experts that were picked.
    torch.testing.assert_close(layer_a(x)[0], layer_b(x)[0])
    assert torch.equal(layer_a.e_expert_biases.detach(), layer_b.e_expert_biases)
    assert layer_b.e_expert_biases.abs().max() > 0
