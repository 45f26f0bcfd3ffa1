"""TensorAccessor: how an op reads from / writes into a slice of a larger buffer.

Follows python/aitemplate/compiler/tensor_accessor.py:32-459 in what the kernels of this path
need: an element `offset` into the base buffer plus one strided dimension (`stride_dim`) whose
trailing extent in the base buffer (`actual_total_elements_from_stride_dim`) differs from the
tensor's own (`original_total_elements_from_stride_dim`). For a GEMM writing into a concat buffer
along the last dim this is exactly (output_offset, output_stride)
(python/aitemplate/backend/cuda/gemm_universal/common.py:36-60).
"""
from __future__ import annotations

import copy
from pprint import pformat
from typing import Any, List, Optional


class TensorAccessor:
    def __init__(self, original_tensor) -> None:
        self.offset = 0
        self.original_shapes = original_tensor._attrs["shape"]
        self.tensor_dtype = original_tensor.dtype()
        self.is_contiguous = True
        self.is_from_strided_tensor = False
        self.stride_dim: Optional[int] = None
        self.actual_shapes = None
        self.original_total_elements_from_stride_dim: Optional[int] = None
        self.actual_total_elements_from_stride_dim: Optional[int] = None

    def __deepcopy__(self, memo):
        res = copy.copy(self)
        res.original_shapes = copy.deepcopy(self.original_shapes, memo)
        res.actual_shapes = copy.deepcopy(self.actual_shapes, memo)
        return res

    def __str__(self) -> str:
        return pformat(vars(self), indent=2)

    __repr__ = __str__

    def __eq__(self, other: Any) -> bool:
        return isinstance(other, TensorAccessor) and vars(self) == vars(other)

    def update_base_tensor(self, new_tensor, stride_dim: int, stride_dim_offset: int) -> None:
        """Makes this accessor address a slice of `new_tensor` that starts `stride_dim_offset`
        elements into dimension `stride_dim` (tensor_accessor.py:349-404). Dims from stride_dim on
        must be static."""
        assert self.stride_dim is None, "accessor already points into a strided buffer"
        orig = self.original_shapes
        new_shape = new_tensor._attrs["shape"]
        assert len(orig) == len(new_shape), "update_base_tensor expects tensors of equal rank"

        def _prod(dims) -> int:
            n = 1
            for d in dims:
                assert len(d._attrs["values"]) == 1, "dims from the stride dim on must be static"
                n *= d._attrs["values"][0]
            return n

        self.stride_dim = stride_dim
        self.original_total_elements_from_stride_dim = _prod(orig[stride_dim:])
        self.actual_total_elements_from_stride_dim = _prod(new_shape[stride_dim:])
        self.offset = stride_dim_offset * _prod(new_shape[stride_dim + 1:])
        self.actual_shapes = new_shape
        self.is_contiguous = False
        self.is_from_strided_tensor = True

    def row_stride(self) -> Optional[int]:
        """Elements between consecutive 'rows' (everything before stride_dim folded), or None."""
        return self.actual_total_elements_from_stride_dim
