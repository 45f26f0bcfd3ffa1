"""Eager, tensor-level access to the kernels of libb200ait through its C ABI.

Each function takes CUDA torch tensors, allocates the output with torch (PyTorch is only used for
device memory and streams) and calls exactly one C entry point on the current stream. The graph
API in aitemplate_b200.compiler reaches the same kernels through the native model container.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_uint8, c_void_p
from typing import List, Optional, Sequence

import torch

from . import _lib

UNARY = {
    "identity": 0, "relu": 1, "gelu": 2, "fast_gelu": 3, "sigmoid": 4, "tanh": 5, "swish": 6, "hardswish": 7,
}
BINARY = {None: 0, "none": 0, "add": 1, "mul": 2}

# name suffix of gemm_rcr_bias_<suffix> -> (u1, b1, b2, u2), following the reference's table
# python/aitemplate/backend/cuda/gemm_universal/gemm_rcr_bias_elementwise.py:34-53
EPILOGUES = {
    "": ("identity", None, None, "identity"),
    "relu": ("relu", None, None, "identity"),
    "gelu": ("gelu", None, None, "identity"),
    "fast_gelu": ("fast_gelu", None, None, "identity"),
    "sigmoid": ("sigmoid", None, None, "identity"),
    "tanh": ("tanh", None, None, "identity"),
    "swish": ("swish", None, None, "identity"),
    "hardswish": ("hardswish", None, None, "identity"),
    "add": ("identity", "add", None, "identity"),
    "add_relu": ("identity", "add", None, "relu"),
    "add_add": ("identity", "add", "add", "identity"),
    "add_add_relu": ("identity", "add", "add", "relu"),
    "mul": ("identity", "mul", None, "identity"),
    "mul_add": ("identity", "mul", "add", "identity"),
    "mul_tanh": ("identity", "mul", None, "tanh"),
    "sigmoid_mul": ("sigmoid", "mul", None, "identity"),
    "sigmoid_mul_tanh": ("sigmoid", "mul", None, "tanh"),
}

EW_OPS = {
    "add": 1, "sub": 2, "mul": 3, "div": 4, "rsub": 5, "rdiv": 6, "max": 7, "min": 8,
    "relu": 16, "gelu": 17, "fast_gelu": 18, "sigmoid": 19, "tanh": 20, "silu": 21, "neg": 22, "abs": 23,
    "exp": 24, "sqrt": 25, "hardswish": 26,
}

_DTYPE_CODE = {torch.float16: 1, torch.bfloat16: 6}


def epilogue_code(name: str) -> int:
    u1, b1, b2, u2 = EPILOGUES[name]
    return UNARY[u1] | (BINARY[b1] << 4) | (BINARY[b2] << 6) | (UNARY[u2] << 8)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    return t.data_ptr() if t.numel() > 0 else None


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}: the kernels take float16 or bfloat16") from None


def _check_cuda(*ts) -> None:
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("tensors must be CUDA tensors")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")


def device_status() -> int:
    """Synchronises and returns the kernel status word (0 = clean), clearing it."""
    out = c_int(0)
    _lib.check(_lib.load().b200ait_device_status(ctypes.byref(out)), "b200ait_device_status")
    return out.value


def gemm_rcr(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    d0: Optional[torch.Tensor] = None,
    d1: Optional[torch.Tensor] = None,
    epilogue: str = "",
    permute_shape: Optional[Sequence[int]] = None,
    permute_layout: str = "20314",
    alpha: float = 1.0,
    tile_n: int = 0,
    out: Optional[torch.Tensor] = None,
    split_k: int = 0,
) -> torch.Tensor:
    """y = epilogue(x @ w.T + bias, d0, d1); x [..., K] (leading dims fold into M), w [N, K].
    split_k: 0 lets the library decide, 1 disables split-K, n allows at most n splits."""
    _check_cuda(x, w, bias, d0, d1)
    if out is not None and not out.is_cuda:
        raise ValueError("tensors must be CUDA tensors")
    if out is not None and not out.is_contiguous() and not (permute_shape is None and out.dim() == 2):
        raise ValueError("tensors must be contiguous")
    k = x.shape[-1]
    m = x.numel() // k if k else math.prod(x.shape[:-1])
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"gemm_rcr: K mismatch {tuple(x.shape)} vs {tuple(w.shape)}")
    store_mode, t1, t2, t3 = 0, 1, 1, 1
    if permute_shape is not None:
        if permute_layout == "20314":
            t1, t2, t3 = permute_shape
            store_mode = 1
            out_shape = [t2, m // t1, t3, t1, n // (t2 * t3)]
        elif permute_layout == "0213":
            t1, t2 = permute_shape
            store_mode = 2
            out_shape = [m // t1, t2, t1, n // t2]
        else:
            raise ValueError(f"unknown permute layout {permute_layout}")
    else:
        out_shape = list(x.shape[:-1]) + [n]
    ldc = n
    if out is None:
        out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    elif store_mode == 0 and out.dim() == 2:
        if out.stride(1) != 1:
            raise ValueError("gemm_rcr: the rows of `out` must be contiguous")
        ldc = out.stride(0)          # a column block of a wider buffer is written in place
    ws = None
    if split_k != 1 and m and n and k:
        ws_bytes = gemm_workspace_bytes(1, m, n, k, tile_n, split_k)
        if ws_bytes:
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    code = _lib.load().b200ait_gemm_rcr(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(d0), _ptr(d1), _ptr(out),
        1, m, n, k, k, k, ldc, n, 0, 0, 0, 0,
        epilogue_code(epilogue), _dtype_code(x), c_float(alpha), store_mode, t1, t2, t3, tile_n,
        _ptr(ws), ws.numel() if ws is not None else 0, split_k, _stream(),
    )
    _lib.check(code, "b200ait_gemm_rcr")
    return out


def gemm_rcr_multi_out(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor],
    out_ptrs: Sequence[int],
    ldc: int,
    d0: Optional[torch.Tensor] = None,
    epilogue: str = "",
    alpha: float = 1.0,
    tile_n: int = 0,
) -> None:
    """epilogue(x @ w.T + bias [, d0]) written to every device address in `out_ptrs` (row stride `ldc`
    elements): this GPU's buffer and peer-mapped pointers to other GPUs' buffers (see sharding.PeerBuffer)."""
    _check_cuda(x, w, bias, d0)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"gemm_rcr_multi_out: K mismatch {tuple(x.shape)} vs {tuple(w.shape)}")
    if not 1 <= len(out_ptrs) <= 8:
        raise ValueError("gemm_rcr_multi_out: 1 to 8 output pointers")
    outs = (c_void_p * len(out_ptrs))(*[c_void_p(int(q)) for q in out_ptrs])
    code = _lib.load().b200ait_gemm_rcr_multi_out(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(d0), outs, len(out_ptrs), m, n, k, k, k, ldc,
        d0.stride(0) if d0 is not None else n, epilogue_code(epilogue), _dtype_code(x), c_float(alpha), tile_n,
        _stream(),
    )
    _lib.check(code, "b200ait_gemm_rcr_multi_out")


def gemm_rrr(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, epilogue: str = "",
             alpha: float = 1.0, tile_n: int = 0) -> torch.Tensor:
    """y = epilogue(x @ w + bias) with w stored [K, N] (row-major B); x [..., K]."""
    _check_cuda(x, w, bias)
    k = x.shape[-1]
    m = x.numel() // k if k else math.prod(x.shape[:-1])
    if w.dim() != 2 or w.shape[0] != k:
        raise ValueError(f"gemm_rrr: K mismatch {tuple(x.shape)} vs {tuple(w.shape)}")
    n = w.shape[1]
    out = torch.empty(list(x.shape[:-1]) + [n], dtype=x.dtype, device=x.device)
    code = _lib.load().b200ait_gemm_rrr(
        _ptr(x), _ptr(w), _ptr(bias), None, None, _ptr(out), 1, m, n, k, k, n, n, n, 0, 0, 0, 0,
        epilogue_code(epilogue), _dtype_code(x), c_float(alpha), tile_n, None, 0, 1, _stream())
    _lib.check(code, "b200ait_gemm_rrr")
    return out


def bmm_rrr(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, tile_n: int = 0) -> torch.Tensor:
    """c[i] = a[i] @ b[i] with a [B, M, K] (or [M, K]) and b [B, K, N] (or [K, N]); batch 1 broadcasts."""
    _check_cuda(a, b)
    a3 = a if a.dim() == 3 else a.unsqueeze(0)
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    ba, m, k = a3.shape
    bb, k2, n = b3.shape
    if k != k2 or not (ba == bb or ba == 1 or bb == 1):
        raise ValueError(f"bmm_rrr: incompatible shapes {tuple(a.shape)} and {tuple(b.shape)}")
    batch = max(ba, bb)
    out = torch.empty((batch, m, n), dtype=a.dtype, device=a.device)
    code = _lib.load().b200ait_gemm_rrr(
        _ptr(a3), _ptr(b3), None, None, None, _ptr(out), batch, m, n, k, k, n, n, n,
        0 if (ba == 1 and batch > 1) else m * k, 0 if (bb == 1 and batch > 1) else n * k, m * n, m * n,
        0, _dtype_code(a), c_float(alpha), tile_n, None, 0, 1, _stream())
    _lib.check(code, "b200ait_gemm_rrr")
    return out


def bmm_permute(a: torch.Tensor, b: torch.Tensor, d1: int, b_row_major: bool = False, alpha: float = 1.0,
                tile_n: int = 0) -> torch.Tensor:
    """bmm_rcr_permute (b [B, N, K]) / bmm_rrr_permute (b [B, K, N], b_row_major): the [B, M, N] product stored as
    [B / d1, d1, M, N].permute(0, 2, 1, 3); returns the [B / d1, M, d1, N] tensor."""
    _check_cuda(a, b)
    a3 = a if a.dim() == 3 else a.unsqueeze(0)
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    ba, m, k = a3.shape
    bb = b3.shape[0]
    k2, n = (b3.shape[1], b3.shape[2]) if b_row_major else (b3.shape[2], b3.shape[1])
    if k != k2 or not (ba == bb or ba == 1 or bb == 1):
        raise ValueError(f"bmm_permute: incompatible shapes {tuple(a.shape)} and {tuple(b.shape)}")
    batch = max(ba, bb)
    if d1 <= 0 or batch % d1:
        raise ValueError(f"bmm_permute: batch {batch} is not a multiple of d1 = {d1}")
    out = torch.empty((batch // d1, m, d1, n), dtype=a.dtype, device=a.device)
    code = _lib.load().b200ait_bmm_permute0213(
        _ptr(a3), _ptr(b3), _ptr(out), batch, m, n, k,
        0 if (ba == 1 and batch > 1) else m * k, 0 if (bb == 1 and batch > 1) else n * k, d1, int(b_row_major),
        _dtype_code(a), c_float(alpha), tile_n, _stream())
    _lib.check(code, "b200ait_bmm_permute0213")
    return out


def gemm_workspace_bytes(batch: int, m: int, n: int, k: int, tile_n: int = 0, split_k: int = 0) -> int:
    """Bytes of fp32 split-K scratch the library would use for this problem (0 = it would not split)."""
    out = c_int64(0)
    _lib.check(_lib.load().b200ait_gemm_rcr_workspace_bytes(batch, m, n, k, tile_n, split_k, ctypes.byref(out)),
               "b200ait_gemm_rcr_workspace_bytes")
    return out.value


def bmm_rcr(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, tile_n: int = 0) -> torch.Tensor:
    """c[i] = a[i] @ b[i].T with a [B, M, K] (or [M, K]) and b [B, N, K] (or [N, K]); batch 1 broadcasts."""
    _check_cuda(a, b)
    a3 = a if a.dim() == 3 else a.unsqueeze(0)
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    ba, m, k = a3.shape
    bb, n, k2 = b3.shape
    if k != k2 or not (ba == bb or ba == 1 or bb == 1):
        raise ValueError(f"bmm_rcr: incompatible shapes {tuple(a.shape)} and {tuple(b.shape)}")
    batch = max(ba, bb)
    out = torch.empty((batch, m, n), dtype=a.dtype, device=a.device)
    code = _lib.load().b200ait_gemm_rcr(
        _ptr(a3), _ptr(b3), None, None, None, _ptr(out),
        batch, m, n, k, k, k, n, n,
        0 if (ba == 1 and batch > 1) else m * k, 0 if (bb == 1 and batch > 1) else n * k, m * n, m * n,
        0, _dtype_code(a), c_float(alpha), 0, 1, 1, 1, tile_n, None, 0, 1, _stream(),
    )
    _lib.check(code, "b200ait_gemm_rcr")
    return out


def mem_eff_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
                      scale: Optional[float] = None, lengths_kv: Optional[torch.Tensor] = None,
                      lengths_q: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [B,H,Sq,D], k [B,H,Skv,D], v [B,H,Skv,Dv] -> [B,Sq,H,Dv]; scale defaults to 1/sqrt(D).
    lengths_kv / lengths_q: int32 device tensors of B values (batch b sees its first lengths_kv[b] keys; only its
    first lengths_q[b] rows are written - pass `out` to choose what the other rows hold)."""
    _check_cuda(q, k, v)
    bsz, h, sq, d = q.shape
    skv, dv = k.shape[2], v.shape[3]
    for name, t in (("lengths_kv", lengths_kv), ("lengths_q", lengths_q)):
        if t is not None and (not t.is_cuda or t.dtype != torch.int32 or t.numel() != bsz or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous int32 GPU tensor with one value per batch")
    if out is None:
        out = torch.empty((bsz, sq, h, dv), dtype=q.dtype, device=q.device)
    elif tuple(out.shape) != (bsz, sq, h, dv) or out.dtype != q.dtype or not out.is_cuda or not out.is_contiguous():
        raise ValueError("out must be a contiguous [B, Sq, H, Dv] GPU tensor of the inputs' dtype")
    if scale is None:
        scale = 1.0 / math.sqrt(d) if d else 1.0
    code = _lib.load().b200ait_mem_eff_attention(
        _ptr(out), _ptr(q), _ptr(k), _ptr(v), bsz, skv, sq, h, d, dv, c_float(scale), int(causal),
        _ptr(lengths_kv) if lengths_kv is not None else None, _ptr(lengths_q) if lengths_q is not None else None,
        _dtype_code(q), _stream(),
    )
    _lib.check(code, "b200ait_mem_eff_attention")
    return out


def _bhsd_strides(t: torch.Tensor):
    """(row, head, batch) element strides of a [B, H, S, D] view; the channel stride must be 1."""
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError("attention operands must be 4-D [B, H, S, D] views with unit channel stride")
    row, head = t.stride(2), t.stride(1)
    batch = t.stride(0) if t.shape[0] > 1 else max(row * t.shape[2], head * t.shape[1])
    return _i64([row, head, batch])


def mem_eff_attention_strided(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
                              scale: Optional[float] = None) -> torch.Tensor:
    """mem_eff_attention on [B, H, S, D] VIEWS that need not be contiguous (e.g. `x.view(B, S, H, D).permute(0, 2,
    1, 3)` of a projection output): the kernel reads them in place through strided tensor maps."""
    for t in (q, k, v):
        if t is not None and not t.is_cuda:
            raise ValueError("inputs must be on GPU")
    bsz, h, sq, d = q.shape
    skv, dv = k.shape[2], v.shape[3]
    out = torch.empty((bsz, sq, h, dv), dtype=q.dtype, device=q.device)
    if scale is None:
        scale = 1.0 / math.sqrt(d) if d else 1.0
    code = _lib.load().b200ait_mem_eff_attention_strided(
        _ptr(out), q.data_ptr(), k.data_ptr(), v.data_ptr(), bsz, skv, sq, h, d, dv, _bhsd_strides(q),
        _bhsd_strides(k), _bhsd_strides(v), c_float(scale), int(causal), _dtype_code(q), _stream(),
    )
    _lib.check(code, "b200ait_mem_eff_attention_strided")
    return out


def flash_attention(qkv: torch.Tensor, cu_seqlens: torch.Tensor, max_seq_len: int, causal: bool = False,
                    scale: Optional[float] = None) -> torch.Tensor:
    """qkv [total, 3, H, D] packed, cu_seqlens int32 [batch + 1] -> [total, H, D]."""
    _check_cuda(qkv, cu_seqlens)
    if cu_seqlens.dtype != torch.int32:
        raise ValueError("cu_seqlens must be int32")
    total, three, h, d = qkv.shape
    if three != 3:
        raise ValueError("qkv must be [total, 3, num_heads, head_size]")
    out = torch.empty((total, h, d), dtype=qkv.dtype, device=qkv.device)
    if scale is None:
        scale = 1.0 / math.sqrt(d) if d else 1.0
    code = _lib.load().b200ait_flash_attention(
        _ptr(out), _ptr(qkv), _ptr(cu_seqlens), None, None, cu_seqlens.numel() - 1, int(max_seq_len), h, d,
        c_float(0.0), c_float(scale), int(causal), 0, total, _dtype_code(qkv), _stream(),
    )
    _lib.check(code, "b200ait_flash_attention")
    return out


def layernorm(x: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor], eps: float = 1e-5,
              normalized_ndim: int = 1) -> torch.Tensor:
    _check_cuda(x, gamma, beta)
    n = math.prod(x.shape[x.dim() - normalized_ndim:])
    m = x.numel() // n if n else 0
    out = torch.empty_like(x)
    code = _lib.load().b200ait_layernorm(
        _ptr(out), _ptr(x), _ptr(gamma), _ptr(beta), m, n, c_float(eps), 0, 0, _dtype_code(x), _stream()
    )
    _lib.check(code, "b200ait_layernorm")
    return out


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    _check_cuda(x)
    dim = dim % x.dim()
    outer = math.prod(x.shape[:dim])
    k = x.shape[dim]
    inner = math.prod(x.shape[dim + 1:])
    out = torch.empty_like(x)
    code = _lib.load().b200ait_softmax(_ptr(x), _ptr(out), outer, k, inner, _dtype_code(x), _stream())
    _lib.check(code, "b200ait_softmax")
    return out


def _i64(vals) -> ctypes.Array:
    return (c_int64 * len(vals))(*[int(v) for v in vals])


def concatenate(tensors: List[torch.Tensor], dim: int = 0, input_masks: Optional[Sequence[bool]] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _check_cuda(*tensors)
    rank = tensors[0].dim()
    dim = dim % rank
    n = len(tensors)
    shape = list(tensors[0].shape)
    shape[dim] = sum(t.shape[dim] for t in tensors)
    if out is None:
        out = torch.empty(shape, dtype=tensors[0].dtype, device=tensors[0].device)
    ptrs = (c_void_p * n)(*[_ptr(t) for t in tensors])
    shapes = [_i64(t.shape) for t in tensors]
    shape_ptrs = (_lib.I64P * n)(*[ctypes.cast(s, _lib.I64P) for s in shapes])
    masks = (c_uint8 * n)(*[1 if (input_masks is None or input_masks[i]) else 0 for i in range(n)])
    out_shape = (c_int64 * rank)()
    code = _lib.load().b200ait_concatenate(
        _ptr(out), out_shape, ptrs, shape_ptrs, masks, dim, rank, n, tensors[0].element_size(), _stream()
    )
    _lib.check(code, "b200ait_concatenate")
    assert list(out_shape) == shape
    return out


def split(x: torch.Tensor, split_size_or_sections, dim: int = 0) -> List[torch.Tensor]:
    _check_cuda(x)
    rank = x.dim()
    dim = dim % rank
    total = x.shape[dim]
    if isinstance(split_size_or_sections, int):
        s = split_size_or_sections
        sizes = [s] * (total // s) + ([total % s] if total % s else []) if s > 0 else []
    else:
        sizes = list(split_size_or_sections)
    outs = []
    for s in sizes:
        shp = list(x.shape)
        shp[dim] = s
        outs.append(torch.empty(shp, dtype=x.dtype, device=x.device))
    n = len(outs)
    ptrs = (c_void_p * n)(*[_ptr(t) for t in outs])
    code = _lib.load().b200ait_split(
        ptrs, None, _ptr(x), _i64(x.shape), n, _i64(sizes), dim, rank, x.element_size(), _stream()
    )
    _lib.check(code, "b200ait_split")
    return outs


def permute(x: torch.Tensor, dims: Sequence[int]) -> torch.Tensor:
    _check_cuda(x)
    dims = [d % x.dim() for d in dims]
    out = torch.empty([x.shape[d] for d in dims], dtype=x.dtype, device=x.device)
    code = _lib.load().b200ait_permute(_ptr(x), _ptr(out), _i64(x.shape), _i64(dims), x.dim(), x.element_size(), _stream())
    _lib.check(code, "b200ait_permute")
    return out


def elementwise(inputs: List[torch.Tensor], steps: Sequence[tuple]) -> torch.Tensor:
    """acc = inputs[0]; each step is (op_name, operand) with operand an input index, a float
    constant, or None for a unary op. Inputs broadcast (torch rules) to the output shape."""
    _check_cuda(*inputs)
    out_shape = list(torch.broadcast_shapes(*[t.shape for t in inputs]))
    rank = len(out_shape)
    out = torch.empty(out_shape, dtype=inputs[0].dtype, device=inputs[0].device)
    n = len(inputs)
    ptrs = (c_void_p * n)(*[_ptr(t) for t in inputs])
    shapes = [_i64([1] * (rank - t.dim()) + list(t.shape)) for t in inputs]
    shape_ptrs = (_lib.I64P * n)(*[ctypes.cast(s, _lib.I64P) for s in shapes])
    ops, operands, consts = [], [], []
    for name, operand in steps:
        ops.append(EW_OPS[name])
        if operand is None:
            operands.append(-2)
            consts.append(0.0)
        elif isinstance(operand, int) and not isinstance(operand, bool):
            operands.append(operand)
            consts.append(0.0)
        else:
            operands.append(-1)
            consts.append(float(operand))
    ns = len(ops)
    code = _lib.load().b200ait_elementwise(
        _ptr(out), _i64(out_shape), rank, ptrs, shape_ptrs, n, (c_int * ns)(*ops), (c_int * ns)(*operands),
        (c_float * ns)(*consts), ns, _dtype_code(inputs[0]), _stream(),
    )
    _lib.check(code, "b200ait_elementwise")
    return out
