"""`from aitemplate_b200.compiler import compile_model, ops, Model` — the reference's
`aitemplate.compiler` surface (python/aitemplate/compiler/__init__.py)."""
from . import base, dtype, ops, tensor_accessor, transform  # noqa: F401
from .base import DynamicProfileStrategy, IntImm, IntVar, IntVarTensor, Operator, Tensor  # noqa: F401
from .compiler import compile_model  # noqa: F401
from .model import AIT_DEFAULT_NUM_RUNTIMES, AITData, AITemplateAllocatorKind, AITemplateMemcpyKind, Model  # noqa: F401

__all__ = ["base", "ops", "transform", "compile_model", "Model", "AITData", "AITemplateAllocatorKind",
           "AITemplateMemcpyKind", "Tensor", "IntVar", "IntImm", "Operator"]
