"""nn front end for the hot path: Module / Parameter plus Linear, LayerNorm, MultiheadAttention,
CrossAttention (python/aitemplate/frontend/nn)."""
from .attention import CrossAttention, MultiheadAttention  # noqa: F401
from .layers import Dropout, Identity, LayerNorm, Linear  # noqa: F401
from .module import Module, ModuleList, Parameter, Sequential  # noqa: F401
