from .elementwise import elementwise, fused_elementwise, fast_gelu, gelu, relu, sigmoid, silu, tanh  # noqa: F401
from .epilogue import EpilogueOp, FuncEnum  # noqa: F401
from .view_ops import flatten, reshape, squeeze, unsqueeze  # noqa: F401
