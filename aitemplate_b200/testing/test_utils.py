"""Small helpers shared by tests and benchmarks (python/aitemplate/testing/test_utils.py:185-188,
python/aitemplate/utils/shape_utils.py:42-51)."""
from __future__ import annotations

from typing import List, Optional, Sequence

from ..compiler.base import IntImm, IntVar


def get_random_torch_tensor(shape, dtype: str = "float16"):
    import torch

    from ..compiler.dtype import string_to_torch_dtype

    return torch.randn(shape, device="cuda", dtype=string_to_torch_dtype(dtype))


def get_torch_empty_tensor(shape, dtype: str = "float16"):
    import torch

    from ..compiler.dtype import string_to_torch_dtype

    return torch.empty(shape, device="cuda", dtype=string_to_torch_dtype(dtype))


def gen_int_var_min_max(values: Sequence[int], name: Optional[str] = None) -> IntVar:
    """IntImm when all values agree, else IntVar([min, max])."""
    lo, hi = min(values), max(values)
    return IntImm(lo, name=name) if lo == hi else IntVar([lo, hi], name=name)


def gen_int_var(values: Sequence[int], name: Optional[str] = None) -> IntVar:
    vals = sorted(set(values))
    return IntImm(vals[0], name=name) if len(vals) == 1 else IntVar(vals, name=name)
