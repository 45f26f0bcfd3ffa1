"""Utilities mirroring python/aitemplate/utils (shape helpers)."""
from . import shape_utils  # noqa: F401
