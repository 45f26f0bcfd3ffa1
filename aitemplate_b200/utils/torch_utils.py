"""torch dtype <-> dtype-string helpers (python/aitemplate/utils/torch_utils.py:30-62)."""
from __future__ import annotations

import torch

_PAIRS = ((torch.float16, "float16"), (torch.bfloat16, "bfloat16"), (torch.float32, "float32"),
          (torch.int32, "int32"), (torch.int64, "int64"), (torch.bool, "bool"))


def torch_dtype_to_string(dtype) -> str:
    for t, s in _PAIRS:
        if dtype == t:
            return s
    raise ValueError(f"Got unsupported input dtype {dtype}! Supported dtypes are: {[s for _, s in _PAIRS]}")


def string_to_torch_dtype(string_dtype):
    if string_dtype is None:
        return None
    aliases = {"half": "float16", "float": "float32", "int": "int32", "long": "int64"}
    string_dtype = aliases.get(string_dtype, string_dtype)
    for t, s in _PAIRS:
        if string_dtype == s:
            return t
    raise ValueError(f"Got unsupported ait dtype {string_dtype}! Supported dtypes are: {[s for _, s in _PAIRS]}")
