"""Pins oracle/reference_ops.py to outputs computed by the REFERENCE's own test-oracle code.

tests/golden/reference_numeric_fixtures.npz was produced by
tests/golden/make_reference_numeric_fixtures.py, which imports the reference's
tests/unittest/ops/test_attention.py and evaluates the cited source lines of the other reference
tests on seeded inputs. Every oracle function the GPU parity tests rely on has to reproduce those
recorded outputs here, so a drift of the restatement from the reference's text fails on CPU.

Not pinned by a reference-computed vector: the tanh form of fast_gelu (the reference's test
compares it with erf-GELU at 1e-1; the tanh constants come from
python/aitemplate/backend/cuda/elementwise/custom_math.cuh:828-851 and are checked against the
closed form in test_oracle_cpu.py).
"""
import os

import numpy as np
import pytest
import torch

from oracle import reference_ops as oracle

FIX = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_numeric_fixtures.npz"))
TOL = 1e-6


def _in(case, name):
    return torch.from_numpy(FIX[f"{case}/in/{name}"])


def _has(case, name):
    return f"{case}/in/{name}" in FIX.files


def _close(got, case, tol=TOL):
    want = torch.from_numpy(FIX[f"{case}/out/y"])
    assert tuple(got.shape) == tuple(want.shape), (case, got.shape, want.shape)
    err = (got.float() - want).abs()
    assert bool((err <= tol + tol * want.abs()).all()), (case, float(err.max()))


GEMM_CASES = {
    "gemm_rcr": "", "gemm_rcr_bias": "", "gemm_rcr_bias_relu": "relu", "gemm_rcr_bias_gelu": "gelu",
    "gemm_rcr_bias_sigmoid": "sigmoid", "gemm_rcr_bias_tanh": "tanh", "gemm_rcr_bias_swish": "swish",
    "gemm_rcr_bias_hardswish": "hardswish", "gemm_rcr_bias_mul_add": "mul_add",
    "gemm_rcr_bias_sigmoid_mul": "sigmoid_mul", "gemm_rcr_bias_sigmoid_mul_tanh": "sigmoid_mul_tanh",
    "gemm_rcr_bias_add": "add", "gemm_rcr_bias_add_relu": "add_relu",
    "gemm_rcr_bias_add_add_relu": "add_add_relu", "gemm_rcr_bias_mul": "mul",
    "gemm_rcr_bias_add_add": "add_add", "gemm_rcr_bias_mul_tanh": "mul_tanh",
}


def test_fixture_covers_every_pinned_case():
    cases = {k.split("/")[0] for k in FIX.files}
    assert set(GEMM_CASES) <= cases
    for c in ("gemm_rrr", "gemm_rcr_bias_permute", "bmm_rcr", "bmm_rrr", "bmm_rrr_permute", "bmm_rcr_permute",
              "layernorm", "layernorm_2d_no_affine", "softmax_dim-1", "softmax_dim1",
              "attention_ref_math_causal0", "attention_ref_math_causal1", "attention_pt", "ref_cross_attention",
              "ref_attention_bmhk", "attention_ref_math_lengths_kv_causal0", "attention_ref_math_lengths_kv_causal1"):
        assert c in cases, c


@pytest.mark.parametrize("case", sorted(GEMM_CASES))
def test_gemm_family_reproduces_reference_outputs(case):
    get = lambda n: _in(case, n) if _has(case, n) else None  # noqa: E731
    got = oracle.gemm_rcr(get("x"), get("w"), get("b"), get("d0"), get("d1"), epilogue=GEMM_CASES[case])
    _close(got, case)


def test_gemm_rrr_reproduces_reference_output():
    _close(oracle.gemm_rrr(_in("gemm_rrr", "x"), _in("gemm_rrr", "w")), "gemm_rrr")


def test_gemm_rcr_bias_permute_20314_reproduces_reference_output():
    c = "gemm_rcr_bias_permute"
    shape = tuple(int(v) for v in _in(c, "shape"))
    _close(oracle.gemm_rcr_bias_permute(_in(c, "x"), _in(c, "w"), _in(c, "b"), shape, "20314"), c)


def test_bmm_family_reproduces_reference_outputs():
    _close(oracle.bmm_rcr(_in("bmm_rcr", "a"), _in("bmm_rcr", "b")), "bmm_rcr")
    _close(oracle.bmm_rrr(_in("bmm_rrr", "a"), _in("bmm_rrr", "b")), "bmm_rrr")
    for c, rrr in (("bmm_rrr_permute", True), ("bmm_rcr_permute", False)):
        _close(oracle.bmm_permute(_in(c, "a"), _in(c, "b"), int(_in(c, "d1")[0]), b_row_major=rrr), c)


def test_layernorm_reproduces_reference_outputs():
    c = "layernorm"
    _close(oracle.layernorm(_in(c, "x"), _in(c, "gamma"), _in(c, "beta"), eps=1e-5), c)
    c = "layernorm_2d_no_affine"
    _close(oracle.layernorm(_in(c, "x"), None, None, eps=1e-12, normalized_ndim=2), c)


def test_softmax_reproduces_reference_outputs():
    for dim in (-1, 1):
        c = f"softmax_dim{dim}"
        _close(oracle.softmax(_in(c, "x"), dim=dim), c)


@pytest.mark.parametrize("causal", [False, True])
def test_attention_reproduces_attention_ref_math(causal):
    c = f"attention_ref_math_causal{int(causal)}"
    qkv = _in(c, "qkv")  # [B, S, 3, H, D]
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))  # -> [B, H, S, D]
    _close(oracle.mem_eff_attention(q, k, v, causal=causal), c, tol=2e-6)  # output [B, S, H, D]


@pytest.mark.parametrize("causal", [False, True])
def test_attention_with_key_lengths_reproduces_attention_ref_math(causal):
    c = f"attention_ref_math_lengths_kv_causal{int(causal)}"
    qkv, lengths = _in(c, "qkv"), _in(c, "lengths_kv")
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    got = oracle.mem_eff_attention(q, k, v, causal=causal, lengths_kv=lengths)
    want = torch.from_numpy(FIX[c + "/out/y"])
    assert torch.equal(torch.isnan(got), torch.isnan(want)) and bool(torch.isnan(want[2]).all())  # the batch without keys
    assert float((got[:2] - want[:2]).abs().max()) <= 2e-6


def test_qkv_permute_plus_attention_reproduces_attention_pt():
    c = "attention_pt"
    nh, d, seq = (int(v) for v in _in(c, "dims"))
    qkv = oracle.gemm_rcr_bias_permute(_in(c, "x"), _in(c, "w"), _in(c, "b"), (seq, 3, nh), "20314")  # [3,1,H,S,D]
    _close(oracle.mem_eff_attention(qkv[0], qkv[1], qkv[2]), c, tol=5e-6)


def test_attention_reproduces_ref_cross_attention():
    c = "ref_cross_attention"  # [B*H, S, D] operands, output [B*H, Sq, D]
    q, k, v = (_in(c, n).unsqueeze(1) for n in "qkv")
    _close(oracle.mem_eff_attention(q, k, v)[:, :, 0, :], c, tol=2e-6)
    c = "ref_attention_bmhk"  # [B, M, H, K] operands, output [B, M, H, K]
    q, k, v = (_in(c, n).permute(0, 2, 1, 3) for n in "qkv")
    _close(oracle.mem_eff_attention(q, k, v), c, tol=2e-6)


def test_bert_layer_is_a_composition_of_pinned_functions():
    """The whole-layer oracle has no counterpart function in the reference; it must equal the
    composition of the pinned single-op oracles."""
    g = torch.Generator().manual_seed(5)
    b, s, hid, heads = 2, 16, 32, 4
    r = lambda *sh, sc=1.0: (torch.randn(*sh, generator=g) * sc).half()  # noqa: E731
    p = {"qkv_weight": r(3 * hid, hid, sc=0.2), "qkv_bias": r(3 * hid, sc=0.2), "proj_weight": r(hid, hid, sc=0.2),
         "proj_bias": r(hid, sc=0.2), "ln1_gamma": r(hid), "ln1_beta": r(hid), "fc1_weight": r(4 * hid, hid, sc=0.2),
         "fc1_bias": r(4 * hid, sc=0.2), "fc2_weight": r(hid, 4 * hid, sc=0.2), "fc2_bias": r(hid, sc=0.2),
         "ln2_gamma": r(hid), "ln2_beta": r(hid)}
    x = r(b, s, hid)
    x2 = x.float().reshape(b * s, hid)
    qkv = oracle.gemm_rcr_bias_permute(x2, p["qkv_weight"], p["qkv_bias"], (s, 3, heads), "20314")
    a = oracle.mem_eff_attention(qkv[0], qkv[1], qkv[2]).reshape(b * s, hid)
    h1 = oracle.layernorm(oracle.gemm_rcr(a, p["proj_weight"], p["proj_bias"], x2, epilogue="add"),
                          p["ln1_gamma"], p["ln1_beta"], eps=1e-12)
    f = oracle.gemm_rcr(h1, p["fc1_weight"], p["fc1_bias"], epilogue="fast_gelu")
    want = oracle.layernorm(oracle.gemm_rcr(f, p["fc2_weight"], p["fc2_bias"], h1, epilogue="add"),
                            p["ln2_gamma"], p["ln2_beta"], eps=1e-12).reshape(b, s, hid)
    got = oracle.bert_layer(x, p, num_heads=heads)
    assert float((got - want).abs().max()) < 1e-5
