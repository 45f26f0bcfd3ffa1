"""`from aitemplate_b200.frontend import Tensor, IntVar, IntImm, nn` (python/aitemplate/frontend/__init__.py)."""
from ..compiler.base import IntImm, IntVar, IntVarTensor, Tensor  # noqa: F401
from . import nn  # noqa: F401
