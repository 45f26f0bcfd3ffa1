"""Shape helpers (python/aitemplate/utils/shape_utils.py:28-120): building IntVar / IntImm dims from
value lists and reading them back."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

from ..compiler.base import IntImm, IntVar


def gen_int_var(values: Sequence[int], name: Optional[str] = None) -> IntVar:
    """IntImm for a single distinct value, else an IntVar over the sorted distinct values
    (shape_utils.py:28-51)."""
    vals = sorted(set(values))
    return IntImm(vals[0], name=name) if len(vals) == 1 else IntVar(vals, name=name)


def gen_int_var_min_max(values: Sequence[int], name: Optional[str] = None) -> IntVar:
    """IntImm when all values agree, else IntVar([min, max]) (shape_utils.py:54-72)."""
    lo, hi = min(values), max(values)
    return IntImm(lo, name=name) if lo == hi else IntVar([lo, hi], name=name)


def convert_shape_to_IntVar(shape: Sequence[Union[int, IntVar]]) -> List[IntVar]:
    """ints become IntImm, IntVars pass through (shape_utils.py:75-97)."""
    out = []
    for d in shape:
        if isinstance(d, IntVar):
            out.append(d)
        elif isinstance(d, int):
            out.append(IntImm(d))
        else:
            raise RuntimeError(f"Unsupported dim type: {type(d)}, dim: {d}")
    return out


def convert_IntVar_to_int(var: Union[IntVar, Sequence[IntVar]]):
    """Static value(s) of IntImm dims; raises for a dynamic dim (shape_utils.py:100-118)."""
    if isinstance(var, (list, tuple)):
        return [convert_IntVar_to_int(v) for v in var]
    vals = var._attrs["values"]
    if len(set(vals)) != 1:
        raise RuntimeError(f"dim {var} is not static")
    return vals[0]


def is_static_dimension(shape: Sequence[IntVar], dim: int) -> bool:
    return -len(shape) <= dim < len(shape) and len(set(shape[dim]._attrs["values"])) == 1


def all_static_dimensions(shape: Sequence[IntVar], from_dim: int = 0) -> bool:
    return all(is_static_dimension(shape, i) for i in range(from_dim, len(shape)))
