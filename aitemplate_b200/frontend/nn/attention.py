"""MultiheadAttention / CrossAttention modules over mem_eff_attention
(python/aitemplate/frontend/nn/attention.py:68-400).

The reference's CUDA default is flash_attention with packed QKV; this build has one attention
kernel, so MultiheadAttention always takes the mem_eff path the reference uses with
`use_mem_eff=True`: QKV projection through gemm_rcr_bias_permute(shape=(seq, 3, heads)) straight
into [3, B, H, S, D], a split on dim 0, mem_eff_attention, and the output projection with the
residual fused (gemm_rcr_bias_add)."""
from __future__ import annotations

from ...compiler import ops
from .layers import Dropout, Linear
from .module import Module


class MultiheadAttention(Module):
    def __init__(self, dim, batch_size, seq_len, num_heads=8, qkv_bias=False, attn_drop=0.0, proj_drop=0.0,
                 has_residual=True, causal=False, mask_seq=0, use_mem_eff=True, dtype="float16"):
        super().__init__()
        assert dim % num_heads == 0, f"dim {dim} should be divisible by num_heads {num_heads}"
        if mask_seq:
            raise NotImplementedError("mask_seq is outside this path")
        self.num_heads = num_heads
        self.scale = (dim // num_heads) ** -0.5
        self.causal = causal
        self.has_residual = has_residual
        self.use_mem_eff = True
        self.op = ops.mem_eff_attention(causal=causal)
        self.qkv = Linear(dim, dim * 3, specialization="permute", shape=(seq_len, 3, num_heads), dtype=dtype)
        self.attn_drop = Dropout(attn_drop, dtype=dtype)
        self.proj = Linear(dim, dim, specialization="add" if has_residual else None, dtype=dtype)
        self.proj_drop = Dropout(proj_drop, dtype=dtype)

    @staticmethod
    def get_shape(x):
        return [d.value() for d in x._attrs["shape"]]

    def qkv_proj(self, x):
        hidden = self.get_shape(x)[-1]
        return self.qkv(ops.reshape()(x, [-1, hidden]))

    def attention(self, x):
        q, k, v = ops.split()(x, 1, dim=0)
        _, b, _, seqlen, d = self.get_shape(q)
        return self.op(ops.reshape()(q, [b, -1, seqlen, d]), ops.reshape()(k, [b, -1, seqlen, d]),
                       ops.reshape()(v, [b, -1, seqlen, d]))

    def forward(self, *args):
        assert len(args) >= 1
        x = args[0]
        batch, seq, hidden = self.get_shape(x)
        attn = self.attention(self.qkv_proj(x))
        attn = ops.reshape()(attn, [batch * seq, -1])
        if self.has_residual:
            assert len(args) == 2
            res = args[1]
            if res._rank() != 2:
                res = ops.reshape()(res, [batch * seq, -1])
            x = self.proj(attn, res)
        else:
            x = self.proj(attn)
        x = self.proj_drop(x)
        return ops.reshape()(x, [batch, seq, hidden])


class CrossAttention(Module):
    def __init__(self, dim, seq_len, seq_len_kv, num_heads, qkv_bias=False, attn_drop=0.0, proj_drop=0.0,
                 has_residual=True, causal=False, dtype="float16"):
        super().__init__()
        assert dim % num_heads == 0, f"dim {dim} should be divisible by num_heads {num_heads}"
        self.num_heads = num_heads
        self.causal = causal
        self.has_residual = has_residual
        self.dim = dim
        self.op = ops.mem_eff_attention(causal=causal)
        self.proj_q = Linear(dim, dim, bias=qkv_bias, dtype=dtype)
        self.proj_k = Linear(dim, dim, bias=qkv_bias, dtype=dtype)
        self.proj_v = Linear(dim, dim, bias=qkv_bias, dtype=dtype)
        self.attn_drop = Dropout(attn_drop, dtype=dtype)
        self.proj = Linear(dim, dim, specialization="add" if has_residual else None, dtype=dtype)
        self.proj_drop = Dropout(proj_drop, dtype=dtype)

    def attention(self, q, k, v):
        batch = q.shape()[0]
        head_dim = self.dim // self.num_heads

        def heads(t, proj):
            return ops.permute()(ops.reshape()(proj(t), [batch, -1, self.num_heads, head_dim]), [0, 2, 1, 3])

        return self.op(heads(q, self.proj_q), heads(k, self.proj_k), heads(v, self.proj_v))

    def forward(self, *args):
        assert len(args) >= 3
        x = args[0]
        batch = x.shape()[0]
        attn = ops.reshape()(self.attention(args[0], args[1], args[2]), [batch, -1, self.dim])
        if self.has_residual:
            assert len(args) == 4
            x = self.proj(attn, args[3])
        else:
            x = self.proj(attn)
        x = self.proj_drop(x)
        return ops.reshape()(x, [batch, -1, self.dim])
