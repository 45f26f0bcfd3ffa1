"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations, and the graphs that run them.

The reference benchmarks BERT-base with HuggingFace weights (examples/03_bert/benchmark_ait.py:263);
no checkpoint is available offline, so weights are drawn from N(0, 0.02) and hidden states from
N(0, 1), generated on the CPU with fixed seeds and rounded to fp16 so that the CPU oracle and the
GPU see identical bits.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..compiler import ops
from ..compiler.base import Tensor
from ..frontend import nn

BERT_BASE = dict(hidden=768, heads=12, ffn=3072, eps=1e-12)


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def bert_layer_inputs(batch: int = 64, seq: int = 384, hidden: int = 768, ffn: int = 3072,
                      seed: int = 1334) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """Returns (hidden_states [batch, seq, hidden] fp16, parameter dict fp16) on the CPU."""
    g = _gen(seed)
    x = torch.randn((batch, seq, hidden), generator=g).half()

    def w(*shape):
        return (torch.randn(shape, generator=g) * 0.02).half()

    params = {
        "qkv_weight": w(3 * hidden, hidden), "qkv_bias": w(3 * hidden),
        "proj_weight": w(hidden, hidden), "proj_bias": w(hidden),
        "ln1_gamma": torch.ones(hidden).half(), "ln1_beta": torch.zeros(hidden).half(),
        "fc1_weight": w(ffn, hidden), "fc1_bias": w(ffn),
        "fc2_weight": w(hidden, ffn), "fc2_bias": w(hidden),
        "ln2_gamma": torch.ones(hidden).half(), "ln2_beta": torch.zeros(hidden).half(),
    }
    return x, params


class BertEncoderLayer(nn.Module):
    """One BERT-base encoder layer built the way the reference builds it
    (examples/03_bert/modeling/bert.py:112-160): MultiheadAttention with the residual fused into the
    output projection, LayerNorm, Linear+fast_gelu, Linear+add, LayerNorm."""

    def __init__(self, batch: int, seq: int, hidden: int = 768, heads: int = 12, ffn: int = 3072,
                 eps: float = 1e-12) -> None:
        super().__init__()
        self.attn = nn.MultiheadAttention(hidden, batch, seq, num_heads=heads, qkv_bias=True, has_residual=True,
                                              use_mem_eff=True)
        self.ln1 = nn.LayerNorm(hidden, eps=eps)
        self.fc1 = nn.Linear(hidden, ffn, specialization="fast_gelu")
        self.fc2 = nn.Linear(ffn, hidden, specialization="add")
        self.ln2 = nn.LayerNorm(hidden, eps=eps)
        self.shape = (batch, seq, hidden)

    def forward(self, x: Tensor) -> Tensor:
        batch, seq, hidden = self.shape
        h = self.attn(x, x)                       # [B, S, hidden], residual = layer input
        h1 = self.ln1(ops.reshape()(h, [batch * seq, hidden]))
        f = self.fc2(self.fc1(h1), h1)
        out = self.ln2(f)
        return ops.reshape()(out, [batch, seq, hidden])


# module parameter name -> key of the dict returned by bert_layer_inputs()
BERT_PARAM_NAMES = {
    "attn_qkv_weight": "qkv_weight", "attn_qkv_bias": "qkv_bias",
    "attn_proj_weight": "proj_weight", "attn_proj_bias": "proj_bias",
    "ln1_weight": "ln1_gamma", "ln1_bias": "ln1_beta",
    "fc1_weight": "fc1_weight", "fc1_bias": "fc1_bias",
    "fc2_weight": "fc2_weight", "fc2_bias": "fc2_bias",
    "ln2_weight": "ln2_gamma", "ln2_bias": "ln2_beta",
}


def build_bert_layer(batch: int = 64, seq: int = 384, hidden: int = 768, heads: int = 12, ffn: int = 3072,
                     eps: float = 1e-12) -> Tuple[Tensor, Tensor]:
    """Builds the graph; returns (input tensor named "hidden_states", output tensor named "output_0")."""
    layer = BertEncoderLayer(batch, seq, hidden, heads, ffn, eps)
    layer.name_parameter_tensor()
    x = Tensor([batch, seq, hidden], name="hidden_states", is_input=True)
    y = layer(x)
    y._attrs["name"] = "output_0"
    y._attrs["is_output"] = True
    return x, y


def bert_layer_flops(batch: int, seq: int, hidden: int = 768, heads: int = 12, ffn: int = 3072) -> float:
    """2MNK per GEMM plus 4 B H S S D for attention (epilogue / softmax flops not counted)."""
    m = batch * seq
    d = hidden // heads
    gemm = 2.0 * m * hidden * (3 * hidden + hidden + ffn + ffn)
    attn = 4.0 * batch * heads * seq * seq * d
    return gemm + attn


# ------------------------------------------------------------------------------------------------
# Stable-Diffusion-style UNet transformer block (latent 64 x 64 = 4096 tokens, dim 320, 8 heads x 40,
# context 77 x 768), built the way the reference builds it
# (examples/05_stable_diffusion/src/modeling/clip.py:42-175: bias-free to_q / to_k / to_v, mem_eff_attention,
# GEGLU as Linear(specialization="mul")(x, Linear(specialization="fast_gelu")(x)), three LayerNorms, each
# sub-block added to its input).

SD_BLOCK = dict(tokens=4096, dim=320, heads=8, head_dim=40, context_tokens=77, context_dim=768, eps=1e-5)


class _SDAttention(nn.Module):
    def __init__(self, batch: int, tokens: int, kv_tokens: int, query_dim: int, context_dim: int, heads: int,
                 head_dim: int) -> None:
        super().__init__()
        inner = heads * head_dim
        self.to_q = nn.Linear(query_dim, inner, bias=False)
        self.to_k = nn.Linear(context_dim, inner, bias=False)
        self.to_v = nn.Linear(context_dim, inner, bias=False)
        self.to_out = nn.Linear(inner, query_dim)
        self.dims = (batch, tokens, kv_tokens, heads, head_dim)

    def forward(self, x: Tensor, context: Tensor, residual: Tensor) -> Tensor:
        batch, tokens, kv_tokens, heads, d = self.dims

        def heads_first(t: Tensor, n: int) -> Tensor:  # [B, n, H*d] -> [B, H, n, d]
            return ops.permute()(ops.reshape()(t, [batch, n, heads, d]), [0, 2, 1, 3])

        q = heads_first(self.to_q(x), tokens)
        k = heads_first(self.to_k(context), kv_tokens)
        v = heads_first(self.to_v(context), kv_tokens)
        out = ops.mem_eff_attention(causal=False)(q, k, v)           # [B, tokens, H, d]
        out = ops.reshape()(out, [batch, tokens, heads * d])
        return self.to_out(out) + residual


class SDTransformerBlock(nn.Module):
    def __init__(self, batch: int, tokens: int = 4096, dim: int = 320, heads: int = 8, head_dim: int = 40,
                 context_tokens: int = 77, context_dim: int = 768, eps: float = 1e-5) -> None:
        super().__init__()
        self.attn1 = _SDAttention(batch, tokens, tokens, dim, dim, heads, head_dim)
        self.attn2 = _SDAttention(batch, tokens, context_tokens, dim, context_dim, heads, head_dim)
        self.norm1 = nn.LayerNorm(dim, eps=eps)
        self.norm2 = nn.LayerNorm(dim, eps=eps)
        self.norm3 = nn.LayerNorm(dim, eps=eps)
        self.ff_proj = nn.Linear(dim, 4 * dim, specialization="mul")
        self.ff_gate = nn.Linear(dim, 4 * dim, specialization="fast_gelu")
        self.ff_out = nn.Linear(4 * dim, dim)

    def forward(self, x: Tensor, context: Tensor) -> Tensor:
        h = self.norm1(x)
        x = self.attn1(h, h, x)
        x = self.attn2(self.norm2(x), context, x)
        h = self.norm3(x)
        return self.ff_out(self.ff_proj(h, self.ff_gate(h))) + x


def sd_block_inputs(batch: int = 2, tokens: int = 4096, dim: int = 320, context_tokens: int = 77,
                    context_dim: int = 768, seed: int = 1534):
    """Returns (x [batch, tokens, dim], context [batch, context_tokens, context_dim], parameters) on the CPU,
    fp16; parameter names are the module parameter names of SDTransformerBlock."""
    g = _gen(seed)
    x = torch.randn((batch, tokens, dim), generator=g).half()
    context = torch.randn((batch, context_tokens, context_dim), generator=g).half()

    def w(*shape):
        return (torch.randn(shape, generator=g) * 0.02).half()

    p = {}
    for name, cdim in (("attn1", dim), ("attn2", context_dim)):
        p[f"{name}_to_q_weight"] = w(dim, dim)
        p[f"{name}_to_k_weight"] = w(dim, cdim)
        p[f"{name}_to_v_weight"] = w(dim, cdim)
        p[f"{name}_to_out_weight"] = w(dim, dim)
        p[f"{name}_to_out_bias"] = w(dim)
    for name in ("norm1", "norm2", "norm3"):
        p[f"{name}_weight"] = torch.ones(dim).half()
        p[f"{name}_bias"] = torch.zeros(dim).half()
    p["ff_proj_weight"], p["ff_proj_bias"] = w(4 * dim, dim), w(4 * dim)
    p["ff_gate_weight"], p["ff_gate_bias"] = w(4 * dim, dim), w(4 * dim)
    p["ff_out_weight"], p["ff_out_bias"] = w(dim, 4 * dim), w(dim)
    return x, context, p


def build_sd_block(batch: int = 2, **kw) -> Tensor:
    """Builds the graph with inputs "latent" [batch, tokens, dim] and "context" [batch, 77, 768]; returns the
    output tensor, named "output_0"."""
    cfg = dict(SD_BLOCK)
    cfg.update(kw)
    block = SDTransformerBlock(batch, cfg["tokens"], cfg["dim"], cfg["heads"], cfg["head_dim"], cfg["context_tokens"],
                               cfg["context_dim"], cfg["eps"])
    block.name_parameter_tensor()
    x = Tensor([batch, cfg["tokens"], cfg["dim"]], name="latent", is_input=True)
    context = Tensor([batch, cfg["context_tokens"], cfg["context_dim"]], name="context", is_input=True)
    y = block(x, context)
    y._attrs["name"] = "output_0"
    y._attrs["is_output"] = True
    return y
