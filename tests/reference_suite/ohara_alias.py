"""pytest plugin that makes ``import ohara...`` resolve to ``ohara_b200...``.

With it the reference project's own test suite runs against this package, which is the most
direct check that the public behaviour matches:

    PYTHONPATH=tests/reference_suite:. python -m pytest -p ohara_alias -p no:cacheprovider \\
        <checkout of the reference>/tests -q

(``tests/test_reference_suite.py`` does exactly that when ``OHARA_REFERENCE_TESTS`` points at the
reference's ``tests`` folder.)"""

import importlib
import importlib.abc
import importlib.util
import sys

_OURS, _THEIRS = "ohara_b200", "ohara"


class _Alias(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path=None, target=None):
        if name != _THEIRS and not name.startswith(_THEIRS + "."):
            return None
        real = _OURS + name[len(_THEIRS):]
        try:
            spec = importlib.util.find_spec(real)
        except ModuleNotFoundError:
            return None
        if spec is None:
            return None
        return importlib.util.spec_from_loader(
            name, self, is_package=spec.submodule_search_locations is not None)

    def create_module(self, spec):
        return importlib.import_module(_OURS + spec.name[len(_THEIRS):])

    def exec_module(self, module):
        """The module is this package's own, already executed."""


if not any(isinstance(finder, _Alias) for finder in sys.meta_path):
    sys.meta_path.insert(0, _Alias())
