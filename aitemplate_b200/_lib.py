"""ctypes binding of libb200ait.so.

There is no CPU or PyTorch fallback: if the library is missing, `load()` raises. The argument
types mirror include/b200ait.h one to one.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint8, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libb200ait.so"

_lock = threading.Lock()
_lib = None

I64P = POINTER(c_int64)
VPP = POINTER(c_void_p)

_GEMM_BIAS = [
    "gemm_rcr_bias", "gemm_rcr_bias_relu", "gemm_rcr_bias_gelu", "gemm_rcr_bias_fast_gelu",
    "gemm_rcr_bias_sigmoid", "gemm_rcr_bias_tanh", "gemm_rcr_bias_swish", "gemm_rcr_bias_hardswish",
]
_GEMM_BIAS_D0 = [
    "gemm_rcr_bias_add", "gemm_rcr_bias_add_relu", "gemm_rcr_bias_mul", "gemm_rcr_bias_mul_tanh",
    "gemm_rcr_bias_sigmoid_mul", "gemm_rcr_bias_sigmoid_mul_tanh",
]
_GEMM_BIAS_D0_D1 = ["gemm_rcr_bias_add_add", "gemm_rcr_bias_add_add_relu", "gemm_rcr_bias_mul_add"]

_DIMS6 = [I64P] * 6


def _signatures():
    sig = {
        "b200ait_last_error": (c_char_p, []),
        "b200ait_version": (c_int, []),
        "b200ait_device_status": (c_int, [POINTER(c_int)]),
        "b200ait_kernel_launch_count": (c_int, [I64P]),
        "b200ait_selftest_bounded_wait": (c_int, [I64P, c_void_p]),
        "b200ait_gemm_rcr": (
            c_int,
            [c_void_p] * 6 + [c_int64] * 12 + [c_int, c_int, c_float, c_int, c_int64, c_int64, c_int64, c_int,
                                               c_void_p, c_int64, c_int, c_void_p],
        ),
        "b200ait_gemm_rcr_workspace_bytes": (c_int, [c_int64] * 4 + [c_int, c_int, I64P]),
        "b200ait_gemm_rrr": (
            c_int,
            [c_void_p] * 6 + [c_int64] * 12 + [c_int, c_int, c_float, c_int, c_void_p, c_int64, c_int, c_void_p],
        ),
        "b200ait_bmm_permute0213": (
            c_int, [c_void_p] * 3 + [c_int64] * 7 + [c_int, c_int, c_float, c_int, c_void_p],
        ),
        "b200ait_gemm_rcr_multi_out": (
            c_int,
            [c_void_p] * 4 + [POINTER(c_void_p), c_int] + [c_int64] * 7 + [c_int, c_int, c_float, c_int, c_void_p],
        ),
        "b200ait_peer_alloc": (c_int, [c_int64, POINTER(c_void_p), c_void_p]),
        "b200ait_peer_open": (c_int, [c_void_p, POINTER(c_void_p)]),
        "b200ait_peer_close": (c_int, [c_void_p]),
        "b200ait_peer_free": (c_int, [c_void_p]),
        "b200ait_gemm_rcr_static_scratch": (
            c_int,
            [c_void_p] * 6 + [c_int64] * 12 + [c_int, c_int, c_float, c_int, c_int64, c_int64, c_int64, c_int,
                                               c_int, c_void_p, c_void_p],
        ),
        "b200ait_gemm_rcr_plain": (c_int, [c_void_p] * 3 + [c_void_p, c_int] + _DIMS6 + [c_void_p]),
        "b200ait_gemm_rcr_bias_permute": (
            c_int,
            [c_void_p] * 4 + [c_void_p, c_int] + _DIMS6 + [c_int64, c_int64, c_int64, c_void_p],
        ),
        "b200ait_bmm_rcr": (c_int, [c_void_p] * 3 + [c_void_p] + [I64P] * 9 + [c_void_p]),
        "b200ait_mem_eff_attention": (
            c_int,
            [c_void_p] * 4 + [c_int64] * 3 + [c_int] * 3 + [c_float, c_int, c_void_p, c_void_p, c_int, c_void_p],
        ),
        "b200ait_mem_eff_attention_strided": (
            c_int,
            [c_void_p] * 4 + [c_int64] * 3 + [c_int] * 3 + [I64P, I64P, I64P, c_float, c_int, c_int, c_void_p],
        ),
        "b200ait_flash_attention": (
            c_int,
            [c_void_p] * 5 + [c_int] * 4 + [c_float, c_float, c_int, c_int, c_int64, c_int, c_void_p],
        ),
        "b200ait_layernorm": (c_int, [c_void_p] * 4 + [c_int64, c_int64, c_float, c_int64, c_int64, c_int, c_void_p]),
        "b200ait_softmax": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
        "b200ait_concatenate": (
            c_int,
            [c_void_p, I64P, VPP, POINTER(I64P), POINTER(c_uint8), c_int64, c_int64, c_int64, c_int64, c_void_p],
        ),
        "b200ait_split": (
            c_int,
            [VPP, POINTER(c_uint8), c_void_p, I64P, c_int64, I64P, c_int64, c_int64, c_int64, c_void_p],
        ),
        "b200ait_permute": (c_int, [c_void_p, c_void_p, I64P, I64P, c_int64, c_int64, c_void_p]),
        "b200ait_elementwise": (
            c_int,
            [c_void_p, I64P, c_int64, VPP, POINTER(I64P), c_int64, POINTER(c_int), POINTER(c_int), POINTER(c_float),
             c_int64, c_int, c_void_p],
        ),
    }
    for n in _GEMM_BIAS:
        sig["b200ait_" + n] = (c_int, [c_void_p] * 4 + [c_void_p, c_int] + _DIMS6 + [c_void_p])
    for n in _GEMM_BIAS_D0:
        sig["b200ait_" + n] = (c_int, [c_void_p] * 5 + [c_void_p, c_int] + _DIMS6 + [c_void_p])
    for n in _GEMM_BIAS_D0_D1:
        sig["b200ait_" + n] = (c_int, [c_void_p] * 6 + [c_void_p, c_int] + _DIMS6 + [c_void_p])
    return sig


def exported_symbols():
    """Names of every per-op entry point include/b200ait.h declares."""
    return sorted(_signatures().keys())


def load() -> ctypes.CDLL:
    """Loads libb200ait.so; raises if it has not been built (there is no fallback path)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m aitemplate_b200.build` "
                "(the CUDA extension is required; there is no CPU fallback)"
            )
        lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_LOCAL)
        for name, (res, args) in _signatures().items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


def kernel_launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    n = c_int64(0)
    check(load().b200ait_kernel_launch_count(ctypes.byref(n)), "b200ait_kernel_launch_count")
    return int(n.value)


def last_error() -> str:
    msg = load().b200ait_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(code: int, what: str) -> None:
    """Turns a non-zero status into RuntimeError, as Model does for the container API
    (python/aitemplate/compiler/model.py:187-198)."""
    if code != 0:
        raise RuntimeError(f"Error in function: {what}: {last_error()}")
