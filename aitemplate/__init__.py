"""`aitemplate`: the reference's import root, answered by aitemplate_b200.

The reference's users write `from aitemplate.compiler import compile_model, ops, Model`,
`from aitemplate.frontend import Tensor, IntVar, nn`, `from aitemplate.testing import detect_target`
(python/aitemplate/compiler/__init__.py, python/aitemplate/compiler/ops/__init__.py:20-37; test idiom
tests/unittest/ops/test_gemm_rcr_bias_fast_gelu.py:72-77). This package makes those statements work
unchanged: every `aitemplate.X.Y` resolves to the module `aitemplate_b200.X.Y` (the same module
object, not a copy), through a meta-path finder installed on import. A submodule that
aitemplate_b200 does not have raises ModuleNotFoundError naming both spellings.
"""
import importlib
import importlib.abc
import importlib.util
import sys

import aitemplate_b200

_PREFIX = __name__ + "."
_TARGET = aitemplate_b200.__name__ + "."


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target):
        self._target = target

    def create_module(self, spec):
        return importlib.import_module(self._target)  # the aliased module object itself

    def exec_module(self, module):  # already executed under its own name
        return None


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(_PREFIX):]
        try:
            found = importlib.util.find_spec(real)
        except ModuleNotFoundError:
            found = None
        if found is None:
            raise ModuleNotFoundError(f"No module named '{fullname}' ('{real}' does not exist either)", name=fullname)
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real), is_package=found.submodule_search_locations is not None)
        return spec


def _install():
    if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, _AliasFinder())


_install()

from aitemplate import backend, compiler, frontend, testing, utils  # noqa: E402,F401

__version__ = aitemplate_b200.__version__
__all__ = ["backend", "compiler", "frontend", "testing", "utils"]
