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
