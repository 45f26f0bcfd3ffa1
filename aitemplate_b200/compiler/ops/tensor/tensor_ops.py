"""Bit-exact data-movement graph nodes: concatenate, split, permute (+ fixed-pattern permutes).

  concatenate  python/aitemplate/compiler/ops/tensor/concatenate.py:33-327
  split        python/aitemplate/compiler/ops/tensor/split.py:26-206 (torch.split semantics, ragged tail)
  permute      python/aitemplate/compiler/ops/tensor/permute.py:35-90 and permute021 / 102 / 210 / 0213
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

from ...base import IntImm, IntVar, Operator, Tensor, wrap_dim
from ...tensor_accessor import TensorAccessor


def _is_empty_rank1(shape: List[IntVar]) -> bool:
    return len(shape) == 1 and shape[0] == IntImm(0)


class concatenate(Operator):
    def __init__(self, fast_cat: bool = True) -> None:
        super().__init__()
        self._attrs["op"] = "concatenate"
        self._attrs["has_profiler"] = False
        self._attrs["fast_cat"] = fast_cat

    def _get_op_attributes(self):
        return {"fast_cat": self._attrs["fast_cat"]}

    def _infer_shapes(self, inputs: List[Tensor], dim: int) -> List[IntVar]:
        if len(inputs) < 1:
            raise RuntimeError("expected a list of Tensors")
        real = [t for t in inputs if not _is_empty_rank1(t._attrs["shape"])]
        if not real:
            return [IntImm(0)]
        rank = real[0]._rank()
        if rank <= 0:
            raise RuntimeError("expected a non-scalar tensor")
        if dim >= rank:
            raise RuntimeError(f"concat_dim ({dim}) expected to be less than rank ({rank})")
        ref = real[0]._attrs["shape"]
        lo = hi = 0
        syms = []
        for t in real:
            s = t._attrs["shape"]
            if len(s) != rank:
                raise RuntimeError(f"tensors expected to have the same rank but got rank={rank} and r={len(s)} "
                                   f"for tensor {t._attrs['name']}")
            for i in range(rank):
                if i != dim and s[i]._attrs["values"] != ref[i]._attrs["values"]:
                    raise RuntimeError(
                        f"tensors expected to have the same dimensions except concat_dim! dim: {i}, "
                        f"shape1: {ref[i]}, shape2: {s[i]}")
            lo += s[dim].lower_bound()
            hi += s[dim].upper_bound()
            syms.append(str(s[dim]._attrs["symbolic_value"]))
        cat = IntImm(lo) if lo == hi else IntVar([lo, hi], symbolic_value="+".join(syms))
        return [cat if i == dim else ref[i] for i in range(rank)]

    def __call__(self, inputs: List[Tensor], dim: int = 0) -> Tensor:
        inputs = list(inputs)
        real = [t for t in inputs if not _is_empty_rank1(t._attrs["shape"])]
        rank = real[0]._rank() if real else 1
        dim = wrap_dim(dim, rank)
        dtypes = {t.dtype() for t in inputs}
        if len(dtypes) > 1:
            raise RuntimeError(f"concatenate: inputs must share one dtype, got {sorted(dtypes)}")
        self._attrs["inputs"] = inputs
        self._attrs["input_accessors"] = [TensorAccessor(t) for t in inputs]
        self._attrs["original_inputs"] = list(inputs)
        self._attrs["input_masks"] = [True] * len(inputs)
        self._attrs["concat_dim"] = dim
        self._set_depth()
        out = Tensor(self._infer_shapes(inputs, dim), src_ops={self}, dtype=inputs[0].dtype())
        self._attrs["outputs"] = [out]
        return out

    def _lower(self) -> Dict[str, Any]:
        masks = [1 if m else 0 for m in self._attrs["input_masks"]]
        return {"kernel": "concatenate", "operands": list(self._attrs["original_inputs"]),
                "ints": [self._attrs["concat_dim"], len(masks)] + masks, "floats": []}


class split(Operator):
    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "split"
        self._attrs["has_profiler"] = False

    def _infer_shapes(self, x: Tensor, split_sizes: List[int], dim: int) -> List[List[IntVar]]:
        x_shape = x._attrs["shape"]
        rank = len(x_shape)
        if rank <= 0:
            raise RuntimeError("expected a non-scalar tensor")
        if dim >= rank:
            raise RuntimeError(f"split dim ({dim}) expected to be less than rank ({rank})")
        if len(split_sizes) < 1:
            raise RuntimeError(f"the number of splits expected >=0 but got {len(split_sizes)}")
        total = x_shape[dim]._attrs["values"][0]
        if sum(split_sizes) != total:
            raise RuntimeError(f"sum of split_sizes ({split_sizes}) does not match split_dim_size ({total})")
        return [list(x_shape[:dim]) + [IntImm(s)] + list(x_shape[dim + 1:]) for s in split_sizes]

    def __call__(self, x: Tensor, split_size_or_sections, dim: int = 0):
        x_shape = x._attrs["shape"]
        self._attrs["inputs"] = [x]
        dim = wrap_dim(dim, x._rank())
        self._attrs["split_dim"] = dim
        self._set_depth()
        if not isinstance(x_shape[dim], IntImm):
            raise NotImplementedError("split dynamic axis")
        if isinstance(split_size_or_sections, (list, tuple)):
            sizes = [s.value() if isinstance(s, IntImm) else int(s) for s in split_size_or_sections]
        else:
            size = split_size_or_sections.value() if isinstance(split_size_or_sections, IntImm) else split_size_or_sections
            if not isinstance(size, int):
                raise RuntimeError("split_size expected to be of int")
            total = x_shape[dim].value()
            if total == 0:
                sizes = [0]
            else:
                if size == 0:
                    raise RuntimeError("split_size expected to be > 0")
                n = (total + size - 1) // size
                sizes = [size] * n
                sizes[-1] = size - (size * n - total)
        self._attrs["split_sizes"] = sizes
        outs = [Tensor(s, src_ops={self}, dtype=x.dtype()) for s in self._infer_shapes(x, sizes, dim)]
        self._attrs["outputs"] = outs
        self._attrs["original_outputs"] = list(outs)
        self._attrs["output_masks"] = [True] * len(outs)
        return tuple(outs)

    def _lower(self) -> Dict[str, Any]:
        sizes = self._attrs["split_sizes"]
        masks = [1 if m else 0 for m in self._attrs["output_masks"]]
        return {"kernel": "split", "operands": [self._attrs["inputs"][0]],
                "ints": [self._attrs["split_dim"], len(sizes)] + list(sizes) + masks, "floats": []}


class _permute_base(Operator):
    def _build(self, x: Tensor, dims: List[int]) -> Tensor:
        self._attrs["inputs"] = [x]
        self._attrs["dims"] = dims
        self._set_depth()
        out = Tensor([x._attrs["shape"][d] for d in dims], src_ops={self}, dtype=x.dtype())
        self._attrs["outputs"] = [out]
        return out

    def _lower(self) -> Dict[str, Any]:
        dims = self._attrs["dims"]
        return {"kernel": "permute", "operands": [self._attrs["inputs"][0]], "ints": [len(dims)] + list(dims), "floats": []}


class permute(_permute_base):
    """permute()(x, dims): torch.permute(x, dims), materialised contiguously."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "permute"

    def __call__(self, x: Tensor, dims: Sequence[int]) -> Tensor:
        dims = [wrap_dim(d, x._rank()) for d in dims]
        sorted_dims = list(range(x._rank()))
        assert sorted(dims) == sorted_dims, f"expected a permutation of {sorted_dims}, but got {dims}"
        self._attrs["dims"] = dims
        # same dispatch to the fixed-pattern ops as the reference (permute.py:64-92); all of them run
        # on the one permute kernel here, the op name is kept for graph-level compatibility
        if dims == [0, 2, 1]:
            return permute021()(x)
        if dims == [1, 0, 2]:
            return permute102()(x)
        if dims == [2, 1, 0]:
            return permute210()(x)
        if dims == [0, 2, 1, 3] and x.shape()[1].lower_bound() >= 24:
            return permute0213()(x)
        if len(dims) > 3 and dims[:-2] + [dims[-1], dims[-2]] == sorted_dims and x.shape()[-1].lower_bound() >= 8:
            return permute021()(x)
        return self._build(x, dims)


def _fixed_permute(name: str, dims: List[int], rank_tail: bool = False):
    def __init__(self) -> None:
        _permute_base.__init__(self)
        self._attrs["op"] = name

    def __call__(self, x: Tensor) -> Tensor:
        r = x._rank()
        if rank_tail:  # permute021 swaps the last two dims of a tensor of any rank >= 3
            assert r >= 3, f"{name} expects rank >= 3"
            d = list(range(r - 2)) + [r - 1, r - 2]
        else:
            assert r == len(dims), f"{name} expects rank {len(dims)}, got {r}"
            d = list(dims)
        return self._build(x, d)

    return type(name, (_permute_base,), {"__init__": __init__, "__call__": __call__,
                                         "__doc__": f"{name}()(x): fixed-pattern permute {dims}."})


permute021 = _fixed_permute("permute021", [0, 2, 1], rank_tail=True)
permute102 = _fixed_permute("permute102", [1, 0, 2])
permute210 = _fixed_permute("permute210", [2, 1, 0])
permute0213 = _fixed_permute("permute0213", [0, 2, 1, 3])
