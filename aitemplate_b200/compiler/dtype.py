"""dtype names, sizes and the AITemplateDtype enum values
(python/aitemplate/compiler/dtype.py:25-157; static/include/model_interface.h:70-78)."""
from __future__ import annotations

_DTYPE_SIZE = {"float16": 2, "bfloat16": 2, "float32": 4, "float": 4, "int32": 4, "int": 4, "int64": 8, "bool": 1}
_ALIASES = {"half": "float16", "float": "float32", "int": "int32", "long": "int64"}
# AITemplateDtype: kUnset=0, kHalf, kFloat, kInt, kLong, kBool, kBFloat16
_DTYPE_TO_ENUM = {"float16": 1, "float32": 2, "float": 2, "int": 3, "int32": 3, "int64": 4, "bool": 5, "bfloat16": 6}
_ENUM_TO_DTYPE = {1: "float16", 2: "float32", 3: "int32", 4: "int64", 5: "bool", 6: "bfloat16"}


def normalize_dtype(dtype: str) -> str:
    dtype = _ALIASES.get(dtype, dtype)
    if dtype not in _DTYPE_SIZE:
        raise KeyError(f"Unknown dtype: {dtype}. Expected one of {sorted(_DTYPE_SIZE)}")
    return dtype


def get_dtype_size(dtype: str) -> int:
    return _DTYPE_SIZE[normalize_dtype(dtype)]


def dtype_str_to_enum(dtype: str) -> int:
    return _DTYPE_TO_ENUM[normalize_dtype(dtype)]


def dtype_enum_to_str(value: int) -> str:
    return _ENUM_TO_DTYPE[value]


def is_same_dtype(a: str, b: str) -> bool:
    return normalize_dtype(a) == normalize_dtype(b)


def torch_dtype_to_string(dtype) -> str:
    import torch

    table = {torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float32: "float32", torch.int32: "int32",
             torch.int64: "int64", torch.bool: "bool"}
    if dtype not in table:
        raise ValueError(f"Got unsupported input dtype {dtype}! Supported dtypes are: {list(table)}")
    return table[dtype]


def string_to_torch_dtype(dtype: str):
    import torch

    table = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32, "int32": torch.int32,
             "int64": torch.int64, "bool": torch.bool}
    return table[normalize_dtype(dtype)]
