"""layernorm graph node (python/aitemplate/compiler/ops/layernorm/layernorm.py:58-450):
`layernorm()(x, gamma, beta, normalized_shape, eps)`; the normalised dims are the trailing static
dims; gamma / beta may be None."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

from ...base import IntImm, IntVar, Operator, Tensor
from ...tensor_accessor import TensorAccessor


class layernorm(Operator):
    def __init__(self, normalized_shape: List[IntImm] = None) -> None:
        super().__init__()
        self._attrs["op"] = "layernorm"
        self._attrs["has_profiler"] = False
        self._attrs["default_normalized_shape"] = normalized_shape
        self._attrs["normalized_shape"] = []
        self._attrs["eps"] = 1e-5
        self._attrs["gamma_constant"] = "1.0"
        self._attrs["beta_constant"] = "0.0"

    def _get_op_attributes(self):
        return {"normalized_shape": self._attrs["default_normalized_shape"]}

    @staticmethod
    def _as_dims(shape) -> List[IntImm]:
        dims = []
        for s in shape:
            if isinstance(s, int):
                dims.append(IntImm(s))
            elif isinstance(s, IntImm):
                dims.append(s)
            else:
                raise NotImplementedError(f"Layernorm normalized_shape must be immediate values. Got {s}")
        return dims

    def _sanity_check(self, x: Tensor, gamma: Optional[Tensor], beta: Optional[Tensor]) -> None:
        ns = self._attrs["normalized_shape"]
        x_shape = x._attrs["shape"]
        if len(ns) == 0 or len(ns) > len(x_shape):
            raise NotImplementedError(f"Layernorm normalized_shape {ns} does not fit input rank {len(x_shape)}")
        if list(x_shape[len(x_shape) - len(ns):]) != list(ns):
            raise RuntimeError(
                f"Layernorm normalized shape is not compatible with input shape. "
                f"Normalized shape: {[d.value() for d in ns]}, input shape: {[d.pseudo_code() for d in x_shape]}")
        for name, t in (("gamma", gamma), ("beta", beta)):
            if t is not None and list(t._attrs["shape"]) != list(ns):
                raise RuntimeError(f"Layernorm {name} shape is not compatible with normalized_shape")

    def __call__(self, x: Tensor, gamma: Tensor = None, beta: Tensor = None, normalized_shape: List[Any] = None,
                 eps: float = 1e-5) -> Tensor:
        inputs = [x]
        self._attrs["gamma_constant"] = "1.0" if gamma is None else None
        self._attrs["beta_constant"] = "0.0" if beta is None else None
        if gamma is not None:
            inputs.append(gamma)
        if beta is not None:
            inputs.append(beta)
        if normalized_shape is None:
            normalized_shape = self._attrs["default_normalized_shape"]
        if normalized_shape is None:
            raise RuntimeError("Layernorm needs a normalized_shape")
        self._attrs["normalized_shape"] = self._as_dims(normalized_shape)
        self._attrs["eps"] = eps
        self._sanity_check(x, gamma, beta)
        self._attrs["inputs"] = inputs
        self._attrs["input_accessors"] = [TensorAccessor(x)]
        self._set_depth()
        out = Tensor(list(x._attrs["shape"]), src_ops={self}, dtype=x.dtype())
        self._attrs["outputs"] = [out]
        self._attrs["output_accessors"] = [TensorAccessor(out)]
        return out

    def _lower(self) -> Dict[str, Any]:
        ins = self._attrs["inputs"]
        x = ins[0]
        idx = 1
        gamma = beta = None
        if self._attrs["gamma_constant"] is None:
            gamma = ins[idx]
            idx += 1
        if self._attrs["beta_constant"] is None:
            beta = ins[idx]
        n = 1
        for d in self._attrs["normalized_shape"]:
            n *= d.value()
        acc = self._attrs["output_accessors"][0]
        out_stride = acc.row_stride() if acc.stride_dim is not None else 0  # 0: contiguous rows of n
        x_acc = self._attrs["input_accessors"][0]
        in_stride = x_acc.row_stride() if x_acc.stride_dim is not None else 0  # rows of a fused split's input
        return {"kernel": "layernorm", "operands": [x, gamma, beta], "ints": [n, acc.offset, out_stride, in_stride],
                "floats": [float(self._attrs["eps"])]}
