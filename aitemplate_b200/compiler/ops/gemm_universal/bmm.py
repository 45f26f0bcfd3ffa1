"""bmm_rcr / bmm_rrr graph nodes: C[b] = alpha * A[b] @ B[b]^T, A [B, M, K], B [B, N, K]
(python/aitemplate/compiler/ops/gemm_universal/bmm.py:69-119, bmm_xxx.py:261-278).
A 2-D operand, or a batch of 1, broadcasts over the other operand's batch."""
from __future__ import annotations

from typing import Any, Dict, List

from ...base import IntImm, IntVar, Tensor
from ...tensor_accessor import TensorAccessor
from .gemm_rcr import gemm


class bmm(gemm):
    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "bmm"

    @staticmethod
    def _batch_dim(a: Tensor, b: Tensor) -> IntVar:
        a_shape, b_shape = a._attrs["shape"], b._attrs["shape"]
        if len(a_shape) == 2:
            return b_shape[0]
        if len(b_shape) == 2:
            return a_shape[0]
        ba, bb = a_shape[0], b_shape[0]
        if ba == IntImm(1):
            return bb
        if bb == IntImm(1) or ba == bb:
            return ba
        raise RuntimeError(f"bmm operand A and B should have same batch_size, or batch_size = 1! "
                           f"Current shape A: {a_shape} shape B: {b_shape} .")

    def _sanity_check(self, a: Tensor, b: Tensor) -> None:
        for name, t in (("A", a), ("B", b)):
            if len(t._attrs["shape"]) not in (2, 3):
                raise RuntimeError(f"bmm operand {name} should have 2 or 3 dimensions! Current shape: {t._attrs['shape']}")
        if len(a._attrs["shape"]) == 2 and len(b._attrs["shape"]) == 2:
            raise RuntimeError("bmm operand A and B both have 2 dimensions! Use gemm instead.")
        if a.dtype() != b.dtype():
            raise RuntimeError("bmm operand A and B should have the same data type!")


class bmm_rcr(bmm):
    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "bmm_rcr"

    def _infer_shapes(self, a: Tensor, b: Tensor) -> List[IntVar]:
        a_shape, b_shape = a._attrs["shape"], b._attrs["shape"]
        if a_shape[-1] != b_shape[-1]:
            raise RuntimeError(f"bmm_rcr operand A and B should have the same K dim! A: {a_shape}, B: {b_shape}")
        return [self._batch_dim(a, b), a_shape[-2], b_shape[-2]]

    def __call__(self, a: Tensor, b: Tensor) -> Tensor:
        self._sanity_check(a, b)
        return self._finish([a, b], self._infer_shapes(a, b))

    def _lower(self) -> Dict[str, Any]:
        a, b = self._attrs["inputs"]
        return {"kernel": "bmm_rcr", "operands": [a, b], "ints": [], "floats": [float(self._attrs["alpha"])]}


class bmm_rrr(bmm):
    """C[b] = alpha * A[b] @ B[b], A [B, M, K], B [B, K, N]
    (python/aitemplate/compiler/ops/gemm_universal/bmm_xxx.py:223-260)."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "bmm_rrr"

    def _infer_shapes(self, a: Tensor, b: Tensor) -> List[IntVar]:
        a_shape, b_shape = a._attrs["shape"], b._attrs["shape"]
        if a_shape[-1] != b_shape[-2]:
            raise RuntimeError(f"bmm_rrr operand A and B should have the same K dim! A: {a_shape}, B: {b_shape}")
        return [self._batch_dim(a, b), a_shape[-2], b_shape[-1]]

    def __call__(self, a: Tensor, b: Tensor) -> Tensor:
        self._sanity_check(a, b)
        return self._finish([a, b], self._infer_shapes(a, b))

    def _lower(self) -> Dict[str, Any]:
        a, b = self._attrs["inputs"]
        return {"kernel": "bmm_rrr", "operands": [a, b], "ints": [], "floats": [float(self._attrs["alpha"])]}
