"""Linear / LayerNorm / Identity / Dropout modules
(python/aitemplate/frontend/nn/linear.py:25-100, layer_norm.py:26-59, identity.py, dropout.py)."""
from __future__ import annotations

from ...compiler import ops
from .module import Module, Parameter


class Linear(Module):
    """y = specialization(x W^T + b). `specialization` names the fused epilogue, e.g. "relu", "gelu",
    "fast_gelu", "add", "add_relu", "mul": the op used is gemm_rcr[_bias][_<specialization>]; epilogues
    with a residual take it as a second forward argument."""

    def __init__(self, in_channels, out_channels, bias=True, specialization=None, dtype="float16", **kwargs):
        super().__init__()
        self.weight = Parameter(shape=[out_channels, in_channels], dtype=dtype)
        op_name = "gemm_rcr_bias" if bias else "gemm_rcr"
        if specialization is not None:
            op_name += "_" + specialization
        if bias:
            self.bias = Parameter(shape=[out_channels], dtype=dtype)
        if not hasattr(ops, op_name):
            raise NotImplementedError(f"{op_name} is not part of this build")
        self._op_name = op_name
        self.op = getattr(ops, op_name)(**kwargs)
        self.use_bias = bias
        self.in_channels = in_channels

    def forward(self, *args):
        assert len(args) >= 1
        inputs = [args[0], self.weight.tensor()]
        if self.use_bias:
            inputs.append(self.bias.tensor())
        inputs.extend(args[1:])
        return self.op(*inputs)


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps=1e-5, dtype="float16", **kwargs):
        super().__init__()
        self.eps = eps
        self.dim = tuple(normalized_shape) if isinstance(normalized_shape, (tuple, list)) else (normalized_shape,)
        self.weight = Parameter(shape=self.dim, dtype=dtype)
        self.bias = Parameter(shape=self.dim, dtype=dtype)
        self.op = ops.layernorm()

    def forward(self, *args):
        assert len(args) == 1
        return self.op(args[0], self.weight.tensor(), self.bias.tensor(), self.dim, self.eps)


class Identity(Module):
    def forward(self, x, *args):
        return x


class Dropout(Identity):
    """Inference only: dropout is the identity (python/aitemplate/frontend/nn/dropout.py)."""

    def __init__(self, p: float = 0.0, **kwargs) -> None:
        super().__init__()
