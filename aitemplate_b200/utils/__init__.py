"""Utilities mirroring python/aitemplate/utils (shape helpers)."""
from . import shape_utils  # noqa: F401


def __getattr__(name):  # torch_utils imports torch: loaded on first use
    if name == "torch_utils":
        import importlib

        return importlib.import_module(__name__ + ".torch_utils")
    raise AttributeError(name)
