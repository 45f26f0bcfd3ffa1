"""MultiheadAttention / CrossAttention modules (python/aitemplate/frontend/nn/attention.py:68-400).

MultiheadAttention keeps the reference's two CUDA paths:
  * default (`use_mem_eff=False`): QKV projection `Linear(dim, 3*dim)`, a reshape to the packed
    [B*S, 3, H, D] layout and `ops.flash_attention` with the module's `cu_length` parameter (the int32
    cumulative sequence offsets, set by the user like any other constant) - attention.py:126-146, 179-186;
  * `use_mem_eff=True`: QKV projection through gemm_rcr_bias_permute(shape=(seq, 3, heads)) straight into
    [3, B, H, S, D], a split on dim 0 and `ops.mem_eff_attention` - attention.py:137-141, 200-208.
Both end in the output projection with the residual fused (gemm_rcr_bias_add). Both attention ops run
the same tensor-core kernel here. Of the reference's third path (bmm_rcr -> softmax -> bmm_rrr_permute
for long sequences at small batch, attention.py:209-224) only the selection heuristic is dropped: the
packed path is taken whenever the head size is one flash_attention accepts, else the mem_eff path."""
from __future__ import annotations

from ...compiler import ops
from .layers import Dropout, Linear
from .module import Module, Parameter


class MultiheadAttention(Module):
    def __init__(self, dim, batch_size, seq_len, num_heads=8, qkv_bias=False, attn_drop=0.0, proj_drop=0.0,
                 has_residual=True, causal=False, mask_seq=0, use_mem_eff=False, dtype="float16"):
        super().__init__()
        assert dim % num_heads == 0, f"dim {dim} should be divisible by num_heads {num_heads}"
        if mask_seq:
            raise NotImplementedError("mask_seq is outside this path")
        self.num_heads = num_heads
        head_dim = dim // num_heads
        self.scale = head_dim ** -0.5
        self.causal = causal
        self.has_residual = has_residual
        self.mask_seq = mask_seq
        self.use_flash = not use_mem_eff and head_dim in {8, 16, 32, 64, 128}
        self.use_mem_eff = not self.use_flash
        if self.use_flash:
            self.op = ops.flash_attention(batch_size=batch_size, dropout=attn_drop, max_seq_len=seq_len, causal=causal)
            self.qkv = Linear(dim, dim * 3, bias=qkv_bias, dtype=dtype)
        else:
            self.op = ops.mem_eff_attention(causal=causal)
            # as in the reference, the permuting projection always carries a bias (attention.py:137-141)
            self.qkv = Linear(dim, dim * 3, specialization="permute", shape=(seq_len, 3, num_heads), dtype=dtype)
        # cu_length: the cumulative sequence lengths, used to index into hidden_states (attention.py:147-148)
        self.cu_length = Parameter(shape=[batch_size + 1], dtype="int32")
        self.attn_drop = Dropout(attn_drop, dtype=dtype)
        self.proj = Linear(dim, dim, specialization="add" if has_residual else None, dtype=dtype)
        self.proj_drop = Dropout(proj_drop, dtype=dtype)

    @staticmethod
    def get_shape(x):
        return [d.value() for d in x._attrs["shape"]]

    def qkv_proj(self, x):
        batch, seq, hidden = self.get_shape(x)
        if self.use_flash:
            return ops.reshape()(self.qkv(x), [int(batch * seq), 3, self.num_heads, hidden // self.num_heads])
        return self.qkv(ops.reshape()(x, [-1, hidden]))

    def attention(self, x):
        if self.use_flash:
            # input [B*S, 3, H, D] -> output [B*S, H, D]
            return self.op(x, self.cu_length.tensor())
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
