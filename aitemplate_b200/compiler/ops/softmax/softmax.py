"""softmax graph node (python/aitemplate/compiler/ops/softmax/softmax.py:76-215):
`softmax()(x, dim)`; the reduction dim and every dim after it must be static."""
from __future__ import annotations

from typing import Any, Dict

from ...base import IntImm, Operator, Tensor, wrap_dim


class softmax(Operator):
    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "softmax"
        self._attrs["has_profiler"] = False
        self._attrs["dim"] = None

    def __call__(self, x: Tensor, dim: int = None) -> Tensor:
        if dim is None:
            raise NotImplementedError("flattening input tensor before normalization is not supported yet")
        if x._rank() < 1:
            raise RuntimeError("softmax needs a tensor of rank >= 1")
        dim = wrap_dim(dim, x._rank())
        for d in x._attrs["shape"][dim:]:
            if not isinstance(d, IntImm):
                raise NotImplementedError(f"softmax requires static dims from the reduction dim on, got {x._attrs['shape']}")
        self._attrs["inputs"] = [x]
        self._attrs["dim"] = dim
        self._set_depth()
        out = Tensor(list(x._attrs["shape"]), src_ops={self}, dtype=x.dtype())
        self._attrs["outputs"] = [out]
        return out

    def _lower(self) -> Dict[str, Any]:
        return {"kernel": "softmax", "operands": [self._attrs["inputs"][0]], "ints": [self._attrs["dim"]], "floats": []}
