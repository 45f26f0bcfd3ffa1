"""Pins the CPU oracle: each expression is checked against an independent restatement of the
formula the reference documents (numpy / explicit loops on small cases), and the blockwise
online-softmax recurrence the kernels use is checked against the direct softmax."""
import math

import numpy as np
import torch

from oracle import reference_ops as oracle


def _rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).half()


def test_fast_gelu_is_the_tanh_form_of_the_reference_kernel():
    # python/aitemplate/backend/cuda/elementwise/custom_math.cuh:828-851
    x = torch.linspace(-6, 6, 1001)
    want = 0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * x * (1 + 0.044715 * x * x)))
    got = oracle._unary("fast_gelu", x)
    assert float((got - want).abs().max()) < 1e-6
    erf = 0.5 * x * (1 + torch.erf(x / math.sqrt(2)))
    assert float((oracle._unary("gelu", x) - erf).abs().max()) < 1e-6
    # the reference's own test compares fast_gelu with erf-GELU at 1e-1: the two forms agree to that
    assert float((got - erf).abs().max()) < 1e-1


def test_gemm_epilogue_table_by_loops():
    x, w, b = _rand((5, 7), 1), _rand((3, 7), 2), _rand((3,), 3)
    d0, d1 = _rand((5, 3), 4), _rand((5, 3), 5)
    base = np.zeros((5, 3), dtype=np.float64)
    for i in range(5):
        for j in range(3):
            base[i, j] = sum(float(x[i, k]) * float(w[j, k]) for k in range(7)) + float(b[j])
    sig = lambda v: 1 / (1 + np.exp(-v))  # noqa: E731
    table = {
        "": base, "relu": np.maximum(base, 0), "add": base + d0.double().numpy(),
        "add_relu": np.maximum(base + d0.double().numpy(), 0),
        "add_add": base + d0.double().numpy() + d1.double().numpy(),
        "mul": base * d0.double().numpy(), "mul_add": base * d0.double().numpy() + d1.double().numpy(),
        "mul_tanh": np.tanh(base * d0.double().numpy()), "sigmoid_mul": sig(base) * d0.double().numpy(),
        "sigmoid_mul_tanh": np.tanh(sig(base) * d0.double().numpy()), "swish": base * sig(base),
    }
    for name, want in table.items():
        _, b1, b2, _ = oracle.EPILOGUES[name]
        got = oracle.gemm_rcr(x, w, b, d0 if b1 else None, d1 if b2 else None, epilogue=name)
        assert np.allclose(got.double().numpy(), want, atol=1e-5), name


def test_permute_20314_index_formula():
    # out[i2, b, i3, s, dd] = y[b*t1 + s, (i2*t3 + i3)*d + dd]
    # (python/aitemplate/compiler/ops/gemm_universal/gemm_rcr_bias_permute.py:59-69)
    t1, t2, t3, d, nb = 4, 3, 2, 5, 2
    x, w, b = _rand((nb * t1, 6), 1), _rand((t2 * t3 * d, 6), 2), _rand((t2 * t3 * d,), 3)
    y = oracle.gemm_rcr(x, w, b)
    p = oracle.gemm_rcr_bias_permute(x, w, b, (t1, t2, t3))
    assert tuple(p.shape) == (t2, nb, t3, t1, d)
    for i2 in range(t2):
        for bb in range(nb):
            for i3 in range(t3):
                for s in range(t1):
                    assert torch.equal(p[i2, bb, i3, s], y[bb * t1 + s, (i2 * t3 + i3) * d:(i2 * t3 + i3 + 1) * d])


def test_attention_blockwise_online_softmax_equals_direct():
    """The recurrence of attention_scaling_coefs_updater.h:85-165 (running max m, running sum l,
    rescale by exp2(m_old - m_new)) restated over key blocks, against the oracle."""
    q, k, v = _rand((2, 3, 37, 16), 1), _rand((2, 3, 53, 16), 2), _rand((2, 3, 53, 8), 3)
    want = oracle.mem_eff_attention(q, k, v)
    qf, kf, vf = q.float(), k.float(), v.float()
    scale_log2 = (1 / math.sqrt(16)) * math.log2(math.e)
    out = torch.zeros(2, 3, 37, 8)
    m = torch.full((2, 3, 37), -float("inf"))
    l = torch.zeros(2, 3, 37)
    for j0 in range(0, 53, 16):
        s = torch.matmul(qf, kf[:, :, j0:j0 + 16].transpose(-1, -2)) * scale_log2
        m_new = torch.maximum(m, s.max(-1).values)
        alpha = torch.exp2(m - m_new)
        p = torch.exp2(s - m_new[..., None])
        l = l * alpha + p.sum(-1)
        out = out * alpha[..., None] + torch.matmul(p, vf[:, :, j0:j0 + 16])
        m = m_new
    got = (out / l[..., None]).permute(0, 2, 1, 3)
    assert float((got - want).abs().max()) < 1e-5
    causal = oracle.mem_eff_attention(q[:, :, :20], k[:, :, :20], v[:, :, :20], causal=True)
    assert torch.allclose(causal[:, 0], v[:, :, 0].float(), atol=1e-6)  # the first query sees only key 0


def test_layernorm_and_softmax_by_formula():
    x, g, b = _rand((6, 33), 1, 3.0), _rand((33,), 2), _rand((33,), 3)
    xf = x.double()
    mean = xf.mean(-1, keepdim=True)
    var = ((xf - mean) ** 2).mean(-1, keepdim=True)
    want = (xf - mean) / torch.sqrt(var + 1e-5) * g.double() + b.double()
    assert float((oracle.layernorm(x, g, b, 1e-5).double() - want).abs().max()) < 1e-5
    e = torch.exp(xf - xf.max(-1, keepdim=True).values)
    assert float((oracle.softmax(x, -1).double() - e / e.sum(-1, keepdim=True)).abs().max()) < 1e-6


def test_bert_layer_oracle_composes_the_op_oracles():
    from aitemplate_b200.testing import workloads

    x, p = workloads.bert_layer_inputs(2, 16, hidden=64, ffn=128)
    heads = 4
    got = oracle.bert_layer(x, p, num_heads=heads)
    m = 2 * 16
    x2 = x.reshape(m, 64)
    qkv = oracle.gemm_rcr_bias_permute(x2, p["qkv_weight"], p["qkv_bias"], (16, 3, heads))
    a = oracle.mem_eff_attention(qkv[0], qkv[1], qkv[2]).reshape(m, 64)
    h1 = oracle.layernorm(oracle.gemm_rcr(a, p["proj_weight"], p["proj_bias"], x2, epilogue="add"),
                          p["ln1_gamma"], p["ln1_beta"], 1e-12)
    f = oracle.gemm_rcr(h1, p["fc1_weight"], p["fc1_bias"], epilogue="fast_gelu")
    want = oracle.layernorm(oracle.gemm_rcr(f, p["fc2_weight"], p["fc2_bias"], h1, epilogue="add"),
                            p["ln2_gamma"], p["ln2_beta"], 1e-12).reshape(2, 16, 64)
    assert float((got - want).abs().max()) < 1e-4


def test_sd_block_oracle_composes_the_op_oracles():
    # the Stable-Diffusion transformer block oracle against its own building blocks, on a small instance
    import math

    import torch
    import torch.nn.functional as F

    from aitemplate_b200.testing import workloads
    from oracle import reference_ops as R

    x, ctx, p = workloads.sd_block_inputs(2, tokens=64, dim=64, context_tokens=9, context_dim=48, seed=5)
    got = R.sd_transformer_block(x, ctx, p, heads=4)

    def attn(name, h, c):
        def heads_first(t):
            b, n, _ = t.shape
            return t.reshape(b, n, 4, 16).permute(0, 2, 1, 3)

        q = heads_first(R.gemm_rcr(h, p[f"{name}_to_q_weight"]))
        k = heads_first(R.gemm_rcr(c, p[f"{name}_to_k_weight"]))
        v = heads_first(R.gemm_rcr(c, p[f"{name}_to_v_weight"]))
        o = R.mem_eff_attention(q, k, v)                       # [B, Sq, H, D]
        o = o.reshape(o.shape[0], o.shape[1], 64)
        return R.gemm_rcr(o, p[f"{name}_to_out_weight"], p[f"{name}_to_out_bias"])

    xf = x.float()
    h = R.layernorm(xf, p["norm1_weight"], p["norm1_bias"])
    xf = attn("attn1", h, h) + xf
    xf = attn("attn2", R.layernorm(xf, p["norm2_weight"], p["norm2_bias"]), ctx.float()) + xf
    h = R.layernorm(xf, p["norm3_weight"], p["norm3_bias"])
    gate = R.gemm_rcr(h, p["ff_gate_weight"], p["ff_gate_bias"], epilogue="fast_gelu")
    ff = R.gemm_rcr(R.gemm_rcr(h, p["ff_proj_weight"], p["ff_proj_bias"]) * gate, p["ff_out_weight"], p["ff_out_bias"])
    want = ff + xf
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
