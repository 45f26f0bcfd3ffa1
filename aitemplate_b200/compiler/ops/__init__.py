"""Graph operators of the fused-GEMM hot path, exported flat like the reference
(python/aitemplate/compiler/ops/__init__.py:20-37): `from aitemplate_b200.compiler import ops`."""
from .attention import *  # noqa: F401,F403
from .common import *  # noqa: F401,F403
from .gemm_universal import *  # noqa: F401,F403
from .layernorm import *  # noqa: F401,F403
from .softmax import *  # noqa: F401,F403
from .tensor import *  # noqa: F401,F403
