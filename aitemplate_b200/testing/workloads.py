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
        self.attn = nn.MultiheadAttention(hidden, batch, seq, num_heads=heads, qkv_bias=True, has_residual=True)
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
