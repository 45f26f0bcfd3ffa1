"""Graph IR: IntVar / IntImm dimensions, Tensor and Operator nodes.

Mirrors the public surface of the reference IR (python/aitemplate/compiler/base.py: IntVar :84-317,
IntImm :319-371, Tensor :728-984, Operator :1104-1274) so that graphs written against
`aitemplate.compiler` build unchanged: every node carries an `_attrs` dict with the same keys the
reference's passes and tests read (shape, name, src_ops, dst_ops, dtype, is_input, is_output,
is_param, is_view_of, value, offset, ...; inputs, outputs, op, depth, ...).
"""
from __future__ import annotations

import copy
import math
from enum import Enum
from numbers import Number
from pprint import pformat
from typing import Any, Dict, Iterable, List, Optional, Sequence, Set, Union

import numpy as np

from .dtype import get_dtype_size, normalize_dtype

__all__ = [
    "Node", "IntVar", "IntImm", "Tensor", "IntVarTensor", "Operator", "DynamicProfileStrategy", "StableSet",
    "get_aligned_size",
]


class StableSet:
    """Insertion-ordered set (python/aitemplate/compiler/stable_set.py): graph traversals must be
    deterministic so that names and memory offsets are reproducible."""

    def __init__(self, items: Optional[Iterable] = None):
        self._d: Dict[Any, None] = {}
        if items is not None:
            for it in items:
                self._d[it] = None

    def add(self, item) -> None:
        self._d[item] = None

    def remove(self, item) -> None:
        del self._d[item]

    def discard(self, item) -> None:
        self._d.pop(item, None)

    def update(self, items: Iterable) -> None:
        for it in items:
            self._d[it] = None

    def clear(self) -> None:
        self._d.clear()

    def __contains__(self, item) -> bool:
        return item in self._d

    def __iter__(self):
        return iter(list(self._d.keys()))

    def __len__(self) -> int:
        return len(self._d)

    def __bool__(self) -> bool:
        return bool(self._d)

    def __getitem__(self, idx):
        return list(self._d.keys())[idx]

    def __eq__(self, other) -> bool:
        if isinstance(other, (StableSet, set, frozenset)):
            return set(self._d.keys()) == set(other)
        return NotImplemented

    def __copy__(self):
        return StableSet(self._d.keys())

    def __repr__(self) -> str:
        return "StableSet(" + repr(list(self._d.keys())) + ")"


class Node:
    """Base of every IR object: a bag of attributes."""

    def __init__(self) -> None:
        self._attrs: Dict[str, Any] = {"name": None, "depth": 0, "nop": False}

    def __str__(self) -> str:
        return pformat(self._attrs, indent=2, depth=2)

    def __repr__(self) -> str:
        return self.__str__()

    def pseudo_code(self, with_shape: bool = False) -> str:
        raise NotImplementedError


_symbol_counter = [0]


def _fresh_symbol(name: Optional[str]) -> str:
    _symbol_counter[0] += 1
    return name if name is not None else f"_sym_{_symbol_counter[0]}"


class IntVar(Node):
    """A dynamic dimension with inclusive bounds [min(values), max(values)].

    Arithmetic returns the most conservative IntVar for the result's range, as the reference
    does (base.py:163-297). Two IntVars are equal when they denote the same symbol.
    """

    def __init__(self, values: List[int], name: Optional[str] = None, symbolic_value: Any = None) -> None:
        super().__init__()
        self._attrs["name"] = name
        if values is None or len(values) < 2:
            raise RuntimeError(f"IntVar 'values' field must have at least 2 values! values: {values}, name: {name}")
        if min(values) < 0:
            raise RuntimeError(f"IntVar has < 0 value! values: {values}, name: {name}")
        vals = sorted(set(int(v) for v in values))
        if len(vals) == 1:
            self._attrs["values"] = vals * 2
            self._attrs["symbolic_value"] = vals[0]
        else:
            self._attrs["values"] = vals
            self._attrs["symbolic_value"] = symbolic_value if symbolic_value is not None else _fresh_symbol(name)

    def __eq__(self, other: Any) -> bool:
        return isinstance(other, IntVar) and self._attrs["symbolic_value"] == other._attrs["symbolic_value"] and \
            self._attrs["values"] == other._attrs["values"]

    def __hash__(self) -> int:
        return hash((self._attrs["name"], tuple(self._attrs["values"]), str(self._attrs["symbolic_value"])))

    def lower_bound(self) -> int:
        return self._attrs["values"][0]

    def upper_bound(self) -> int:
        return self._attrs["values"][-1]

    def symbolic_value(self):
        return self._attrs["symbolic_value"]

    def pseudo_code(self, with_shape: bool = False) -> str:
        return self._attrs["name"] if self._attrs["name"] is not None else f"IntVar({self._attrs['values']})"

    # ---- arithmetic on ranges
    @staticmethod
    def _bounds(x) -> tuple:
        if isinstance(x, IntVar):
            return x.lower_bound(), x.upper_bound(), x._attrs["symbolic_value"]
        if isinstance(x, int):
            return x, x, x
        raise NotImplementedError(f"unsupported operand for IntVar arithmetic: {type(x)}")

    @staticmethod
    def _make(lo: int, hi: int, sym) -> "IntVar":
        if lo == hi:
            return IntImm(lo)
        return IntVar([max(lo, 0), max(hi, 0)], symbolic_value=sym)

    def __add__(self, other):
        a, b, s = self._bounds(self)
        c, d, t = self._bounds(other)
        return self._make(a + c, b + d, f"({s}+{t})")

    __radd__ = __add__

    def __sub__(self, other):
        a, b, s = self._bounds(self)
        c, d, t = self._bounds(other)
        return self._make(a - d, b - c, f"({s}-{t})")

    def __rsub__(self, other):
        a, b, s = self._bounds(self)
        c, d, t = self._bounds(other)
        return self._make(c - b, d - a, f"({t}-{s})")

    def __mul__(self, other):
        a, b, s = self._bounds(self)
        c, d, t = self._bounds(other)
        return self._make(a * c, b * d, f"({s}*{t})")

    __rmul__ = __mul__

    def __truediv__(self, other):
        a, b, s = self._bounds(self)
        c, d, t = self._bounds(other)
        return self._make(a // max(d, 1), b // max(c, 1), f"({s}/{t})")

    def __rtruediv__(self, other):
        a, b, s = self._bounds(self)
        c, d, t = self._bounds(other)
        return self._make(c // max(b, 1), d // max(a, 1), f"({t}/{s})")


class IntImm(IntVar):
    """A static dimension."""

    def __init__(self, value: int, name: Optional[str] = None) -> None:
        if not isinstance(value, (int, np.integer)) or isinstance(value, bool):
            raise RuntimeError(f"IntImm only takes an int value! Name: {name}, current value: {value}")
        Node.__init__(self)
        self._attrs["name"] = name
        self._attrs["values"] = [int(value)]
        self._attrs["symbolic_value"] = int(value)

    def __eq__(self, other: Any) -> bool:
        if isinstance(other, int):
            return self.value() == other
        return isinstance(other, IntImm) and self._attrs["values"] == other._attrs["values"]

    def __hash__(self) -> int:
        return hash(("IntImm", self._attrs["values"][0]))

    def value(self) -> int:
        return self._attrs["values"][0]

    def pseudo_code(self, with_shape: bool = False) -> str:
        return str(self.value())


def get_aligned_size(shape: List[IntVar], dtype: str, alignment: int = 64) -> int:
    """Bytes of a tensor at the upper bound of every dim, rounded up to `alignment`
    (python/aitemplate/compiler/base.py:600-622)."""
    size = get_dtype_size(dtype)
    for v in shape:
        size *= v.upper_bound()
    return (size + alignment - 1) // alignment * alignment if alignment > 1 else size


class _ConstantData:
    """Bytes bound to a constant tensor at compile time (python/aitemplate/compiler/base.py:625-726)."""

    def __init__(self, raw: bytes, dtype: str) -> None:
        self._raw = raw
        self.dtype = normalize_dtype(dtype)

    def to_bytes(self) -> bytes:
        return self._raw

    def size(self) -> int:
        return len(self._raw)

    def is_dtype(self, dtype: str) -> bool:
        return normalize_dtype(dtype) == self.dtype

    def __len__(self) -> int:
        return self.size()


def _as_constant_data(data) -> _ConstantData:
    if isinstance(data, _ConstantData):
        return data
    if isinstance(data, np.ndarray):
        return _ConstantData(np.ascontiguousarray(data).tobytes(), str(data.dtype))
    try:
        import torch

        if isinstance(data, torch.Tensor):
            t = data.detach().contiguous().cpu()
            from .dtype import torch_dtype_to_string

            return _ConstantData(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"", torch_dtype_to_string(t.dtype))
    except ImportError:  # pragma: no cover
        pass
    raise TypeError(f"cannot bind constant data of type {type(data)}")


class Tensor(Node):
    """A value flowing between operators."""

    def __init__(
        self,
        shape: List[Union[int, IntVar]],
        name: Optional[str] = None,
        src_ops: Optional[Iterable["Operator"]] = None,
        dst_ops: Optional[Iterable["Operator"]] = None,
        dtype: str = "float16",
        is_input: bool = False,
        is_output: bool = False,
        value: Any = None,
        is_view_of: Any = None,
        is_internal_constant: bool = False,
        skip_constant_folding: bool = False,
        check_nan_and_inf: bool = False,
        check_outputs: bool = False,
        original_name: Optional[str] = None,
    ) -> None:
        super().__init__()
        self._attrs["shape"] = self._convert_shape(shape)
        self._attrs["name"] = name
        self._attrs["src_ops"] = StableSet(src_ops)
        self._attrs["dst_ops"] = StableSet(dst_ops)
        self._attrs["dtype"] = normalize_dtype(dtype)
        self._attrs["is_output"] = is_output
        self._attrs["is_input"] = is_input
        self._attrs["is_param"] = False
        self._attrs["is_internal_constant"] = is_internal_constant
        self._attrs["skip_constant_folding"] = skip_constant_folding
        self._attrs["has_output_aliases"] = False
        self._attrs["external_tensor"] = None
        self._attrs["is_view_of"] = is_view_of
        if is_view_of is not None:
            self._attrs["dtype"] = is_view_of._attrs["dtype"]
        self._attrs["value"] = value
        depths = [op._attrs["depth"] for op in self._attrs["src_ops"]]
        self._attrs["depth"] = max(depths) + 1 if depths else 0
        self._attrs["offset"] = None
        self._attrs["data"] = None
        self._attrs["constant_folding_output_idx"] = None
        self._attrs["check_nan_and_inf"] = check_nan_and_inf
        self._attrs["check_outputs"] = check_outputs
        self._attrs["original_name"] = original_name

    def __str__(self) -> str:
        out = {}
        for k, v in self._attrs.items():
            if k in ("src_ops", "dst_ops") and v is not None:
                out[k] = [x._attrs["name"] for x in v]
            elif k == "is_view_of" and v is not None:
                out[k] = v._attrs["name"]
            else:
                out[k] = v
        return pformat(out, indent=2)

    @staticmethod
    def _convert_shape(shape) -> List[IntVar]:
        ret = []
        for v in shape:
            if isinstance(v, (int, np.integer)) and not isinstance(v, bool):
                ret.append(IntImm(int(v)))
            elif isinstance(v, IntVar):
                ret.append(v)
            else:
                raise RuntimeError(f"Unsupported dim type: {type(v)}, dim: {v}")
        return ret

    def shape(self) -> List[IntVar]:
        return self._attrs["shape"]

    def _rank(self) -> int:
        return len(self._attrs["shape"])

    def _size(self, dim: int) -> IntVar:
        return self._attrs["shape"][wrap_dim(dim, self._rank())]

    def dtype(self) -> str:
        return self._attrs["dtype"]

    def src_ops(self) -> StableSet:
        return self._attrs["src_ops"]

    def dst_ops(self) -> StableSet:
        return self._attrs["dst_ops"]

    def is_a_const_num(self) -> bool:
        return len(self._attrs["shape"]) == 0 and self._attrs["value"] is not None

    def is_jagged(self) -> bool:
        return False

    def size_bytes(self, alignment: int = 1) -> int:
        return get_aligned_size(self._attrs["shape"], self.dtype(), alignment)

    def pseudo_code(self, with_shape: bool = True) -> str:
        name = self._attrs["name"] or "None"
        if not with_shape:
            return f"(Tensor(name={name}))"
        dims = ", ".join(d.pseudo_code() for d in self._attrs["shape"])
        return f"(Tensor(name={name}, shape=[{dims}]))"

    def _bind_data(self, data) -> None:
        """Binds constant bytes (python/aitemplate/compiler/base.py:924-950)."""
        if self._attrs["src_ops"]:
            raise ValueError(f"Cannot bind tensor {self._attrs['name']}; it has src_ops")
        data = _as_constant_data(data)
        if not data.is_dtype(self.dtype()):
            raise ValueError(f"data's dtype did not match: expected {self.dtype()}, got {data.dtype}")
        need = self.size_bytes(alignment=1)
        if need != len(data):
            raise ValueError(f"ConstantTensor's maximum size is not equal to len(data)! Got {len(data)=}, but expected at least {need} bytes.")
        self._attrs["data"] = data

    def __deepcopy__(self, memo):
        result = Tensor(self._attrs["shape"])
        memo[id(self)] = result
        result._attrs = copy.deepcopy(self._attrs, memo)
        return result

    # elementwise sugar (python/aitemplate/compiler/base.py:958-984)
    def _ew(self, func_name: str, a, b):
        from .ops.common.elementwise import elementwise
        from .ops.common.epilogue import FuncEnum

        return elementwise(FuncEnum[func_name])(a, b)

    def __add__(self, other):
        return self._ew("ADD", self, other)

    def __radd__(self, other):
        return self._ew("ADD", other, self)

    def __sub__(self, other):
        return self._ew("SUB", self, other)

    def __rsub__(self, other):
        return self._ew("SUB", other, self)

    def __mul__(self, other):
        return self._ew("MUL", self, other)

    def __rmul__(self, other):
        return self._ew("MUL", other, self)

    def __truediv__(self, other):
        return self._ew("DIV", self, other)

    def __rtruediv__(self, other):
        return self._ew("DIV", other, self)

    def __neg__(self):
        return self._ew("MUL", -1, self)


class IntVarTensor(Tensor):
    """A tensor that stands for a single dynamic dimension (python/aitemplate/compiler/base.py:1007-1079),
    used to pass a dim into reshape."""

    def __init__(self, int_var: IntVar, name: Optional[str] = None, src_ops=None, dst_ops=None,
                 dtype: str = "float16", is_input: bool = False, is_output: bool = False, value: Any = None,
                 is_view_of: Any = None) -> None:
        super().__init__([], name, src_ops, dst_ops, dtype=dtype, is_input=is_input, is_output=is_output)
        self._attrs["int_var"] = int_var
        self._attrs["symbolic_value"] = int_var._attrs["symbolic_value"]

    def pseudo_code(self, with_shape: bool = True) -> str:
        return f"IntVarTensor({self._attrs['int_var'].pseudo_code()})"


class DynamicProfileStrategy(Enum):
    """Which size of a dynamic M the compile-time GEMM profiler times (python/aitemplate/compiler/base.py:1081-1093):
    MAX the upper bound (default), MIN the lower bound; HINTS is treated as MAX."""

    MIN = 1
    MAX = 2
    HINTS = 3


def wrap_dim(idx: int, rank: int) -> int:
    """Normalises a possibly negative dim index (python/aitemplate/compiler/ops/common/... wrap_dim)."""
    assert isinstance(idx, int), f"dim must be an int, got {type(idx)}"
    if idx < 0:
        idx += rank
    assert 0 <= idx < rank, f"dim {idx} out of range for rank {rank}"
    return idx


class Operator(Node):
    """Base class of graph operators. Calling an operator performs shape inference and links the
    output tensor(s) into the graph."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["inputs"] = None
        self._attrs["outputs"] = None
        self._attrs["has_profiler"] = False

    def __call__(self, *args, **kwargs):
        raise NotImplementedError

    def _set_depth(self) -> None:
        """Depth = 1 + max input depth; registers this op as a consumer of its inputs."""
        depth = 0
        for t in self._attrs["inputs"] or []:
            depth = max(depth, t._attrs["depth"])
            t._attrs["dst_ops"].add(self)
        self._attrs["depth"] = depth

    def __deepcopy__(self, memo):
        result = type(self)(**self._get_op_attributes())
        memo[id(self)] = result
        result._attrs = copy.deepcopy(self._attrs, memo)
        return result

    def __str__(self) -> str:
        out = {}
        for k, v in self._attrs.items():
            if k in ("inputs", "args", "outputs", "original_inputs") and v is not None:
                out[k] = [x._attrs["name"] for x in v]
            else:
                out[k] = v
        return pformat(out, indent=2)

    def replace_input_tensor(self, old_tensor: Tensor, new_tensor: Tensor) -> None:
        self._attrs["inputs"] = [new_tensor if t is old_tensor else t for t in self._attrs["inputs"]]
        if "args" in self._attrs and self._attrs["args"] is not None:
            self._attrs["args"] = [new_tensor if t is old_tensor else t for t in self._attrs["args"]]

    def _get_op_attributes(self) -> Dict[str, Any]:
        """Constructor kwargs needed to clone this op."""
        return {}

    # ---- hooks the reference exposes; no per-model code generation happens here
    def gen_profiler(self, workdir=None, dynamic_profiling_strategy=None) -> None:
        return None

    def profile(self, workdir="./", devices=None, dynamic_profiling_strategy=DynamicProfileStrategy.MAX) -> None:
        return None

    def gen_function(self) -> str:
        raise NotImplementedError(
            "kernels are prebuilt in libb200ait.so; ops lower to plan entries (see Operator._lower)")

    def _lower(self) -> Dict[str, Any]:
        """Returns {"kernel": str, "ints": [...], "floats": [...]} consumed by the native executor."""
        raise NotImplementedError(f"op {self._attrs.get('op')} has no lowering")

    def _inputs_for_pseudo_code(self):
        return self._attrs["inputs"]

    def _outputs_for_pseudo_code(self):
        return self._attrs["outputs"]

    def _args_for_pseudo_code(self):
        return [f"{k}={v}" for k, v in self._get_op_attributes().items()]

    def pseudo_code(self, with_shape: bool = True) -> str:
        args = ",\n".join(t.pseudo_code(with_shape) for t in self._inputs_for_pseudo_code())
        outs = ", ".join(t.pseudo_code(with_shape) for t in self._outputs_for_pseudo_code())
        name = self._attrs.get("name", None)
        return f"# {name}\n{outs} \n= {self._attrs['op']}({', '.join(self._args_for_pseudo_code())})(\n{args})\n"
