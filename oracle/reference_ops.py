"""CPU oracle for the fused-GEMM hot path. TEST INFRASTRUCTURE ONLY.

This module restates, in fp32 PyTorch on the host, the expressions the reference's own unit tests
use as ground truth for each op of the path. It is imported only by tests/, by
__graft_entry__.smoke() and by bench.py's cpu_baseline / --impl reference legs, always as the
checker or the timed CPU baseline and never by the product path (aitemplate_b200/ never imports it).

Pinning. The reference ships no golden vectors for these ops: every one of its tests compares the
compiled kernel with a PyTorch expression on the same inputs. Each function below restates that
expression (file:line per function), in fp32 on inputs first rounded to fp16, and is PINNED to the
reference's own text: tests/golden/make_reference_numeric_fixtures.py imports the reference's
tests/unittest/ops/test_attention.py (attention_ref_math, attention_pt, ref_cross_attention,
ref_attention_bmhk) and evaluates the cited source lines of the other reference tests on seeded
inputs; tests/test_oracle_pinned_cpu.py requires every function here to reproduce those recorded
outputs to 1e-6. Not pinned by a reference-computed vector: the tanh form of fast_gelu
(test_gemm_rcr_bias_fast_gelu.py compares with erf-GELU at atol=rtol=1e-1, so below 1e-1 the tanh
form is pinned by the kernel source custom_math.cuh:828-851 only), and the whole-block functions
bert_layer / sd_transformer_block, which are checked to equal the composition of the pinned
single-op functions. tests/golden/ additionally holds fixtures produced by importing the
reference's Python graph layer (shape inference and op attributes).

Inputs may be fp16/bf16/fp32 tensors on any device; they are moved to the CPU and up-cast.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().to("cpu", torch.float32)


# ------------------------------------------------------------------------------- gemm family
def _unary(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "identity":
        return x
    if name == "relu":  # tests/unittest/ops/test_gemm_bias_relu.py:64-65
        return torch.relu(x)
    if name == "gelu":  # tests/unittest/ops/test_gemm_rcr_bias_fast_gelu.py:96 (torch.nn.GELU())
        return F.gelu(x)
    if name == "fast_gelu":  # python/aitemplate/backend/cuda/elementwise/custom_math.cuh:828-851 (tanh form)
        return F.gelu(x, approximate="tanh")
    if name == "sigmoid":  # tests/unittest/ops/test_gemm_bias_sigmoid.py
        return torch.sigmoid(x)
    if name == "tanh":  # tests/unittest/ops/test_gemm_bias_tanh.py
        return torch.tanh(x)
    if name == "swish":  # tests/unittest/ops/test_gemm_bias_swish.py (x * sigmoid(x))
        return x * torch.sigmoid(x)
    if name == "hardswish":  # tests/unittest/ops/test_gemm_bias_hardswish.py
        return F.hardswish(x)
    raise KeyError(name)


# (u1, b1, b2, u2) per op-name suffix: python/aitemplate/backend/cuda/gemm_universal/gemm_rcr_bias_elementwise.py:34-53
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


def gemm_rcr(x, w, bias=None, d0=None, d1=None, epilogue: str = "", alpha: float = 1.0) -> torch.Tensor:
    """F.linear(X, W, bias) then the epilogue: tests/unittest/ops/test_gemm_bias.py:69,
    test_gemm_bias_relu.py:64-65, test_gemm_rcr_bias_fast_gelu.py:96, test_gemm_bias_broadcast.py:216-219."""
    x, w, bias, d0, d1 = map(_f32, (x, w, bias, d0, d1))
    y = F.linear(x, w) * alpha
    if bias is not None:
        y = y + bias
    u1, b1, b2, u2 = EPILOGUES[epilogue]
    y = _unary(u1, y)
    if b1 == "add":
        y = y + d0
    elif b1 == "mul":
        y = y * d0
    if b2 == "add":
        y = y + d1
    elif b2 == "mul":
        y = y * d1
    return _unary(u2, y)


def gemm_rrr(x, w, bias=None) -> torch.Tensor:
    """tests/unittest/ops/test_gemm.py (rrr case) / test_gemm_bias.py: torch.matmul(X, W) [+ bias], W stored [K, N]."""
    x, w, bias = map(_f32, (x, w, bias))
    y = torch.matmul(x, w)
    return y if bias is None else y + bias


def bmm_rrr(a, b, alpha: float = 1.0) -> torch.Tensor:
    """tests/unittest/ops/test_bmm.py: torch.bmm(A, B), B stored [batch, K, N]."""
    a, b = _f32(a), _f32(b)
    if a.dim() == 2:
        a = a.unsqueeze(0)
    if b.dim() == 2:
        b = b.unsqueeze(0)
    return torch.matmul(a, b) * alpha


def bmm_permute(a, b, d1: int, b_row_major: bool = False, alpha: float = 1.0) -> torch.Tensor:
    """tests/unittest/ops/test_bmm_permute.py: Y = bmm(A, B^T) (rcr) or bmm(A, B) (rrr), then
    Y.reshape(B // D1, D1, M, N).permute(0, 2, 1, 3)."""
    y = bmm_rrr(a, b, alpha) if b_row_major else bmm_rcr(a, b, alpha)
    bsz, m, n = y.shape
    return y.reshape(bsz // d1, d1, m, n).permute(0, 2, 1, 3).contiguous()


def gemm_rcr_bias_permute(x, w, bias, shape: Sequence[int], layout: str = "20314") -> torch.Tensor:
    """tests/unittest/ops/test_gemm_bias_permute.py:74-75 and test_attention.py:146-149:
    linear -> reshape [M/t1, t1, t2, t3, N/t2/t3] -> permute (2, 0, 3, 1, 4)."""
    y = gemm_rcr(x, w, bias)
    m, n = y.shape
    if layout == "20314":
        t1, t2, t3 = shape
        return y.reshape(m // t1, t1, t2, t3, n // (t2 * t3)).permute(2, 0, 3, 1, 4).contiguous()
    if layout == "0213":
        t1, t2 = shape
        return y.reshape(m // t1, t1, t2, n // t2).permute(0, 2, 1, 3).contiguous()
    raise KeyError(layout)


def bmm_rcr(a, b, alpha: float = 1.0) -> torch.Tensor:
    """tests/unittest/ops/test_bmm.py:50-51: torch.bmm(X, W.transpose(2, 1))."""
    a, b = _f32(a), _f32(b)
    if a.dim() == 2:
        a = a.unsqueeze(0)
    if b.dim() == 2:
        b = b.unsqueeze(0)
    batch = max(a.shape[0], b.shape[0])
    a = a.expand(batch, -1, -1)
    b = b.expand(batch, -1, -1)
    return torch.bmm(a, b.transpose(2, 1)) * alpha


# --------------------------------------------------------------------------------- attention
def mem_eff_attention(q, k, v, causal: bool = False, scale: Optional[float] = None, lengths_kv=None,
                      lengths_q=None) -> torch.Tensor:
    """tests/unittest/ops/test_attention.py:111-139 (attention_ref_math) and :167-193
    (ref_cross_attention): softmax(q (k/sqrt d)^T) v with q, k, v [B,H,S,D]; output [B,Sq,H,Dv].
    lengths_kv [B]: batch b sees its first lengths_kv[b] keys (test_attention.py:504-530 builds the same key mask
    for attention_ref); a batch without keys comes out NaN, which that test accepts (equal_nan) and the reference
    kernel produces (0 / 0, kernel_forward.h:833). lengths_q [B]: rows from lengths_q[b] on are not computed by the
    reference (kernel_forward.h:187-192; the test zeroes them on both sides): they are returned as NaN here so that a
    comparison has to leave them out."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    d = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    sq, skv = s.shape[-2], s.shape[-1]
    if causal:
        mask = torch.ones(sq, skv, dtype=torch.bool).tril()
        s = s.masked_fill(~mask, float("-inf"))
    if lengths_kv is not None:
        seen = torch.arange(skv)[None, :] < torch.as_tensor(lengths_kv).reshape(-1, 1).cpu()  # [B, Skv]
        s = s.masked_fill(~seen[:, None, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)  # a row of -inf only: NaN
    o = torch.matmul(p, v)
    o = o.permute(0, 2, 1, 3).contiguous()
    if lengths_q is not None:
        rows = torch.arange(sq)[None, :] < torch.as_tensor(lengths_q).reshape(-1, 1).cpu()      # [B, Sq]
        o = o.masked_fill(~rows[:, :, None, None], float("nan"))
    return o


# ------------------------------------------------------------------------ layernorm / softmax
def layernorm(x, gamma=None, beta=None, eps: float = 1e-5, normalized_ndim: int = 1) -> torch.Tensor:
    """tests/unittest/ops/test_layernorm.py:122: F.layer_norm(x, normalized_shape, gamma, beta, eps)."""
    x, gamma, beta = _f32(x), _f32(gamma), _f32(beta)
    ns = tuple(x.shape[x.dim() - normalized_ndim:])
    return F.layer_norm(x, ns, gamma, beta, eps)


def softmax(x, dim: int = -1) -> torch.Tensor:
    """tests/unittest/ops/test_softmax.py:85: F.softmax(x, dim)."""
    return F.softmax(_f32(x), dim=dim)


# ---------------------------------------------------------------------------- bit-exact ops
def concatenate(tensors: List[torch.Tensor], dim: int = 0) -> torch.Tensor:
    """tests/unittest/ops/test_concatenate.py:74: torch.cat, compared with torch.equal."""
    return torch.cat([t.detach().cpu() for t in tensors], dim=dim)


def split(x: torch.Tensor, split_size_or_sections, dim: int = 0) -> List[torch.Tensor]:
    """tests/unittest/ops/test_split.py:107: torch.split, compared with torch.equal."""
    return [t.contiguous() for t in torch.split(x.detach().cpu(), split_size_or_sections, dim=dim)]


def permute(x: torch.Tensor, dims: Sequence[int]) -> torch.Tensor:
    """tests/unittest/ops/test_permute.py: torch.permute(x, dims).contiguous()."""
    return x.detach().cpu().permute(*dims).contiguous()


_EW = {
    "add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b, "div": lambda a, b: a / b,
    "rsub": lambda a, b: b - a, "rdiv": lambda a, b: b / a, "max": torch.maximum, "min": torch.minimum,
    "relu": lambda a, _: torch.relu(a), "gelu": lambda a, _: F.gelu(a),
    "fast_gelu": lambda a, _: F.gelu(a, approximate="tanh"), "sigmoid": lambda a, _: torch.sigmoid(a),
    "tanh": lambda a, _: torch.tanh(a), "silu": lambda a, _: F.silu(a), "neg": lambda a, _: -a,
    "abs": lambda a, _: a.abs(), "exp": lambda a, _: a.exp(), "sqrt": lambda a, _: a.sqrt(),
    "hardswish": lambda a, _: F.hardswish(a),
}


def elementwise(inputs: List[torch.Tensor], steps: Sequence[tuple]) -> torch.Tensor:
    """tests/unittest/ops/test_fused_elementwise.py: the torch expression of the same chain, in fp32."""
    ins = [_f32(t) for t in inputs]
    acc = ins[0]
    for name, operand in steps:
        if operand is None:
            b = None
        elif isinstance(operand, int) and not isinstance(operand, bool):
            b = ins[operand]
        else:
            b = torch.tensor(float(operand))
        acc = _EW[name](acc, b)
    shape = torch.broadcast_shapes(*[t.shape for t in ins])
    return acc.expand(shape).contiguous()


# ------------------------------------------------------------------------- whole-block oracles
def bert_layer(hidden, p: dict, num_heads: int = 12, eps: float = 1e-12) -> torch.Tensor:
    """One BERT-base encoder layer as examples/03_bert/modeling/bert.py:112-160 builds it with
    nn.MultiheadAttention(use_mem_eff=True) (python/aitemplate/frontend/nn/attention.py:96-286)."""
    h = _f32(hidden)
    b, s, hid = h.shape
    d = hid // num_heads
    w = {k: _f32(v) for k, v in p.items()}
    x = h.reshape(b * s, hid)
    qkv = F.linear(x, w["qkv_weight"], w["qkv_bias"]).reshape(b, s, 3, num_heads, d).permute(2, 0, 3, 1, 4)
    q, k, v = qkv[0], qkv[1], qkv[2]
    a = torch.softmax(torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(d), dim=-1) @ v
    a = a.permute(0, 2, 1, 3).reshape(b * s, hid)
    h1 = F.layer_norm(F.linear(a, w["proj_weight"], w["proj_bias"]) + x, (hid,), w["ln1_gamma"], w["ln1_beta"], eps)
    f = F.gelu(F.linear(h1, w["fc1_weight"], w["fc1_bias"]), approximate="tanh")
    out = F.layer_norm(F.linear(f, w["fc2_weight"], w["fc2_bias"]) + h1, (hid,), w["ln2_gamma"], w["ln2_beta"], eps)
    return out.reshape(b, s, hid)


def sd_transformer_block(x, context, p: dict, heads: int = 8, eps: float = 1e-5) -> torch.Tensor:
    """Stable-Diffusion UNet BasicTransformerBlock as examples/05_stable_diffusion/src/modeling/clip.py:137-175
    builds it: x += attn1(norm1(x)); x += attn2(norm2(x), context); x += ff(norm3(x)), with bias-free q/k/v
    projections (clip.py:59-61) and a GEGLU feed-forward, proj(x) * gelu_tanh(gate(x)) (clip.py:100-107)."""
    x, context = _f32(x), _f32(context)
    w = {k: _f32(v) for k, v in p.items()}
    b, n, dim = x.shape
    d = dim // heads

    def attention(name, h, ctx):
        def split_heads(t):
            return t.reshape(b, -1, heads, d).permute(0, 2, 1, 3)

        q = split_heads(F.linear(h, w[f"{name}_to_q_weight"]))
        k = split_heads(F.linear(ctx, w[f"{name}_to_k_weight"]))
        v = split_heads(F.linear(ctx, w[f"{name}_to_v_weight"]))
        a = torch.softmax(torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(d), dim=-1) @ v
        a = a.permute(0, 2, 1, 3).reshape(b, n, dim)
        return F.linear(a, w[f"{name}_to_out_weight"], w[f"{name}_to_out_bias"])

    def norm(name, t):
        return F.layer_norm(t, (dim,), w[f"{name}_weight"], w[f"{name}_bias"], eps)

    h = norm("norm1", x)
    x = attention("attn1", h, h) + x
    x = attention("attn2", norm("norm2", x), context) + x
    h = norm("norm3", x)
    gate = F.gelu(F.linear(h, w["ff_gate_weight"], w["ff_gate_bias"]), approximate="tanh")
    ff = F.linear(F.linear(h, w["ff_proj_weight"], w["ff_proj_bias"]) * gate, w["ff_out_weight"], w["ff_out_bias"])
    return ff + x
