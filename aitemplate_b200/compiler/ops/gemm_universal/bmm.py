"""bmm_rcr / bmm_rrr graph nodes: C[b] = alpha * A[b] @ B[b]^T, A [B, M, K], B [B, N, K]
(python/aitemplate/compiler/ops/gemm_universal/bmm.py:69-119, bmm_xxx.py:261-278).
A 2-D operand, or a batch of 1, broadcasts over the other operand's batch."""
from __future__ import annotations

from typing import Any, Dict, List, Tuple

from ...base import IntImm, IntVar, Tensor
from ...tensor_accessor import TensorAccessor
from ..common.view_ops import reshape
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

    def _plan_ints(self) -> List[int]:
        """[d1, lda, ldb, out_offset, ldc]: d1 of a "0213" permuted store (bmm_*_permute; 0 = plain [B, M, N]);
        row strides of A and B when they are column blocks of a wider buffer (a split read in place; 0 =
        contiguous); element offset and row stride of the output when it is a column block of a concatenate's
        buffer (0 stride = contiguous). The batch strides follow as rows x row stride."""
        acc_a, acc_b = self._attrs["input_accessors"][:2]
        out = self._attrs["output_accessors"][0]
        return [int(self._attrs.get("permute_d1", 0)),
                acc_a.row_stride() if acc_a.stride_dim is not None else 0,
                acc_b.row_stride() if acc_b.stride_dim is not None else 0,
                out.offset, out.row_stride() if out.stride_dim is not None else 0]

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
        return {"kernel": "bmm_rcr", "operands": [a, b], "ints": self._plan_ints(),
                "floats": [float(self._attrs["alpha"])]}


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
        return {"kernel": "bmm_rrr", "operands": [a, b], "ints": self._plan_ints(),
                "floats": [float(self._attrs["alpha"])]}


def _permute_variant(base, op_name: str):
    """bmm whose [B, M, N] result is stored as [B / d1, d1, M, N].permute(0, 2, 1, 3); returns that 4-D tensor
    [B / d1, M, d1, N] (python/aitemplate/compiler/ops/gemm_universal/bmm_rcr_permute.py:28-116 and
    bmm_rrr_permute.py; epilogue layout Permute4DBMM_0213)."""

    def __init__(self, shape: Tuple[int, ...], layout: str = "0213") -> None:
        base.__init__(self)
        if layout != "0213":
            raise NotImplementedError(f"{layout} is not implemented!")
        self._attrs["op"] = op_name
        self._attrs["shape"] = tuple(shape)
        self._attrs["layout"] = f"Permute4DBMM_{layout}"
        self._attrs["permute_shape"] = "_".join(map(str, shape))
        self._attrs["permute_d1"] = int(shape[0])

    def _get_op_attributes(self):
        return {"layout": self._attrs["layout"].split("_")[-1], "shape": self._attrs["shape"]}

    def __call__(self, a: Tensor, b: Tensor) -> Tensor:
        out = base.__call__(self, a, b)
        batch, m, n = out._attrs["shape"]
        d1 = self._attrs["permute_d1"]
        if not isinstance(batch, IntImm) or d1 <= 0 or batch.value() % d1:
            raise RuntimeError(f"{op_name}: the batch ({batch}) must be static and a multiple of shape[0] = {d1}")
        return reshape()(out, [batch.value() // d1, m, d1, n])

    return type(op_name, (base,), {"__init__": __init__, "__call__": __call__,
                                   "_get_op_attributes": _get_op_attributes, "__doc__": _permute_variant.__doc__})


bmm_rcr_permute = _permute_variant(bmm_rcr, "bmm_rcr_permute")
bmm_rrr_permute = _permute_variant(bmm_rrr, "bmm_rrr_permute")
