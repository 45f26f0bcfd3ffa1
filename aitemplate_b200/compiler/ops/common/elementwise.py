"""elementwise(FuncEnum) graph node with numpy-style broadcasting.

Same construction idiom as the reference (python/aitemplate/compiler/ops/common/elementwise.py:165-296):
`ops.elementwise(FuncEnum.ADD)(x, y)`; Python scalars become rank-0 constant tensors kept in
`_attrs["args"]` while `_attrs["inputs"]` lists only real tensors.
"""
from __future__ import annotations

from typing import Any, Dict, List

from ...base import IntImm, IntVar, Operator, Tensor
from .epilogue import FuncEnum

# FuncEnum -> (kernel op code, arity); codes are those of b200ait_elementwise (include/b200ait.h)
_BINARY = {FuncEnum.ADD: 1, FuncEnum.SUB: 2, FuncEnum.MUL: 3, FuncEnum.DIV: 4, FuncEnum.MAX: 7, FuncEnum.MIN: 8}
_REVERSED = {FuncEnum.ADD: 1, FuncEnum.MUL: 3, FuncEnum.MAX: 7, FuncEnum.MIN: 8, FuncEnum.SUB: 5, FuncEnum.DIV: 6}
_UNARY = {
    FuncEnum.RELU: 16, FuncEnum.GELU: 17, FuncEnum.FASTGELU: 18, FuncEnum.SIGMOID: 19, FuncEnum.TANH: 20,
    FuncEnum.SILU: 21, FuncEnum.ABS: 23, FuncEnum.EXP: 24, FuncEnum.SQRT: 25,
}


def broadcast_shapes(shapes: List[List[IntVar]]) -> List[IntVar]:
    """Right-aligned broadcasting over IntVar shapes (elementwise.py:68-87)."""
    rank = max(len(s) for s in shapes)
    out: List[IntVar] = []
    for i in range(rank):
        dim = None
        for s in shapes:
            j = i - (rank - len(s))
            if j < 0:
                continue
            d = s[j]
            if dim is None or dim == IntImm(1):
                dim = d
            elif d == IntImm(1) or d == dim:
                continue
            elif isinstance(d, IntImm) and isinstance(dim, IntImm):
                raise RuntimeError(f"Tensor shapes are not broadcastable: {shapes}")
            elif isinstance(d, IntImm) and not isinstance(dim, IntImm):
                dim = d  # a static size pins a dynamic one
        out.append(dim)
    return out


def elementwise_steps(func: FuncEnum, args: List[Tensor], inputs: List[Tensor]):
    """Lowers one elementwise node to accumulator steps: returns (ordered_inputs, steps) where steps
    are (op_code, operand_index | -1 const | -2 none, constant)."""
    if func in _UNARY:
        assert len(args) == 1, f"{func} takes one argument"
        return [args[0]], [(_UNARY[func], -2, 0.0)]
    if func not in _BINARY:
        raise NotImplementedError(f"elementwise {func} is outside the fused-GEMM hot path")
    assert len(args) == 2, f"{func} takes two arguments"
    a, b = args
    if a.is_a_const_num() and b.is_a_const_num():
        raise NotImplementedError("elementwise on two constants")
    if b.is_a_const_num():
        return [a], [(_BINARY[func], -1, float(b._attrs["value"]))]
    if a.is_a_const_num():
        return [b], [(_REVERSED[func], -1, float(a._attrs["value"]))]
    return [a, b], [(_BINARY[func], 1, 0.0)]


class elementwise(Operator):
    def __init__(self, func_enum: FuncEnum) -> None:
        super().__init__()
        self._attrs["op"] = "elementwise"
        self._attrs["func"] = func_enum
        self._attrs["has_profiler"] = False

    def _infer_shapes(self, *args: Tensor) -> List[IntVar]:
        return broadcast_shapes([a._attrs["shape"] for a in args])

    def __call__(self, *args) -> Tensor:
        assert len(args) > 0, "Elementwise ops must take at least one argument."
        converted = []
        dtype = None
        for a in args:
            if isinstance(a, (int, float)) and not isinstance(a, bool):
                converted.append(Tensor(shape=[], value=a))
            elif isinstance(a, Tensor):
                converted.append(a)
                if dtype is None:
                    dtype = a.dtype()
                elif a.dtype() != dtype:
                    raise NotImplementedError(
                        f"Type promotions are not supported; got dtype {a.dtype()}, but expected {dtype}")
            else:
                raise RuntimeError(f"Unsupported data type {a} in elementwise {self}!")
        dtype = dtype or "float16"
        for a in converted:
            if a.is_a_const_num():
                a._attrs["dtype"] = dtype
        self._attrs["args"] = list(converted)
        self._attrs["inputs"] = [a for a in converted if not a.is_a_const_num()]
        self._set_depth()
        out = Tensor(self._infer_shapes(*converted), src_ops={self}, dtype=dtype)
        self._attrs["outputs"] = [out]
        return out

    def _get_op_attributes(self) -> Dict[str, Any]:
        return {"func_enum": self._attrs["func"]}

    def replace_input_tensor(self, old_tensor, new_tensor) -> None:
        super().replace_input_tensor(old_tensor, new_tensor)

    def _args_for_pseudo_code(self):
        return [f"func={self._attrs['func']}"]

    def _lower(self) -> Dict[str, Any]:
        ordered, steps = elementwise_steps(self._attrs["func"], self._attrs["args"], self._attrs["inputs"])
        return {"kernel": "elementwise", "inputs": ordered, "steps": steps}


class fused_elementwise(Operator):
    """A linear chain of elementwise ops executed by one kernel launch
    (python/aitemplate/compiler/ops/common/fused_elementwise.py:34-127). Built by the
    fuse_elementwise pass from `elementwise` nodes; `_attrs["elementwise_ops"]` keeps the originals."""

    def __init__(self, elementwise_ops: List[elementwise], inputs: List[Tensor], outputs: List[Tensor],
                 steps=None) -> None:
        super().__init__()
        self._attrs["op"] = "fused_elementwise"
        self._attrs["elementwise_ops"] = list(elementwise_ops)
        self._attrs["inputs"] = list(inputs)
        self._attrs["outputs"] = list(outputs)
        self._attrs["steps"] = steps
        self._attrs["has_profiler"] = False
        self._set_depth()
        for t in outputs:
            t._attrs["src_ops"] = type(t._attrs["src_ops"])([self])

    def _get_op_attributes(self):
        return {"elementwise_ops": self._attrs["elementwise_ops"], "inputs": self._attrs["inputs"],
                "outputs": self._attrs["outputs"], "steps": self._attrs["steps"]}

    def _lower(self) -> Dict[str, Any]:
        return {"kernel": "elementwise", "inputs": self._attrs["inputs"], "steps": self._attrs["steps"]}


def _elementwise_func(func_enum: FuncEnum, *args) -> Tensor:
    return elementwise(func_enum)(*args)


# functional helpers exported as ops.tanh(x), ops.relu(x), ... (python/aitemplate/compiler/ops/common/math.py)
def tanh(x):
    return _elementwise_func(FuncEnum.TANH, x)


def relu(x):
    return _elementwise_func(FuncEnum.RELU, x)


def sigmoid(x):
    return _elementwise_func(FuncEnum.SIGMOID, x)


def gelu(x):
    return _elementwise_func(FuncEnum.GELU, x)


def fast_gelu(x):
    return _elementwise_func(FuncEnum.FASTGELU, x)


def silu(x):
    return _elementwise_func(FuncEnum.SILU, x)
