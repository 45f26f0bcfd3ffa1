"""Generates tests/golden/reference_numeric_fixtures.npz: seeded inputs and the outputs that the
REFERENCE's own test-oracle code computes for them.

Nothing is restated here. Two routes, both evaluate the reference's text:
  * functions: tests/unittest/ops/test_attention.py is imported as a module (with the reference's
    python package on the path) and its attention_ref_math / attention_pt / ref_cross_attention are
    called;
  * one-liners: the cited source lines of a reference test file are read from that file, dedented,
    `self.` stripped, and exec'd in a namespace that holds the seeded inputs under the variable
    names the test uses.

Run in a container that has the reference checkout (needs no GPU):
    AIT_BUILD_DOCS=1 PYTHONPATH=<reference>/python \
        python tests/golden/make_reference_numeric_fixtures.py <reference>
AIT_BUILD_DOCS makes the reference's detect_target() return a target without a GPU
(python/aitemplate/testing/detect_target.py:116-118). The fixtures are consumed by
tests/test_oracle_pinned_cpu.py, which requires oracle/reference_ops.py to reproduce every output.

Inputs are stored as fp16 (the reference tests draw fp16 tensors); the reference expressions are
evaluated on their fp32 up-casts so that the recorded outputs do not depend on the host's fp16
matmul kernels. Outputs are stored as fp32.
"""
import importlib.util
import os
import sys
import textwrap
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def rnd(shape, seed, scale=1.0, uniform=False):
    g = torch.Generator().manual_seed(seed)
    t = (torch.rand(shape, generator=g) * 2 - 1) if uniform else torch.randn(shape, generator=g)
    return (t * scale).half()


def exec_reference_lines(ref_root, rel_path, first, last, namespace):
    """Evaluates lines first..last (1-based, inclusive) of a reference file in `namespace`."""
    with open(os.path.join(ref_root, rel_path)) as f:
        lines = f.readlines()[first - 1:last]
    text = textwrap.dedent("".join(lines)).replace("self.", "")
    exec(compile(text, f"{rel_path}:{first}-{last}", "exec"), namespace)
    return text


def import_reference_attention_tests(ref_root):
    """Imports tests/unittest/ops/test_attention.py of the reference. `parameterized` is not
    installed here; only its decorator is used by the test classes, never by the oracle functions,
    so a pass-through stand-in is enough."""
    if "parameterized" not in sys.modules:
        stub = types.ModuleType("parameterized")

        class _P:
            @staticmethod
            def expand(*a, **k):
                return lambda fn: fn

        stub.parameterized = _P
        stub.param = lambda *a, **k: (a, k)
        sys.modules["parameterized"] = stub
    path = os.path.join(ref_root, "tests/unittest/ops/test_attention.py")
    spec = importlib.util.spec_from_file_location("reference_test_attention", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    import aitemplate

    assert os.path.abspath(aitemplate.__file__).startswith(os.path.abspath(ref_root)), \
        "this script must import the reference package"
    out = {}
    texts = {}

    def put(case, inputs, outputs):
        for k, v in inputs.items():
            out[f"{case}/in/{k}"] = v.numpy()
        for k, v in outputs.items():
            out[f"{case}/out/{k}"] = v.detach().float().contiguous().numpy()

    U = "tests/unittest/ops/"

    # ---- the gemm_rcr_bias family: (case, file, [(first, last), ...] evaluated in order, uses d0, uses d1)
    x, w, b = rnd((24, 40), 1), rnd((16, 40), 2, 0.3), rnd((16,), 3)
    d0, d1 = rnd((24, 16), 4), rnd((24, 16), 24)
    B = "test_gemm_bias_broadcast.py"
    gemm_cases = [
        ("gemm_rcr", "test_gemm.py", [(69, 69)], 0, 0, False),
        ("gemm_rcr_bias", "test_gemm_bias.py", [(69, 69)], 0, 0, True),
        ("gemm_rcr_bias_relu", "test_gemm_bias_relu.py", [(64, 65)], 0, 0, True),
        ("gemm_rcr_bias_gelu", "test_gemm_rcr_bias_fast_gelu.py", [(96, 96)], 0, 0, True),
        ("gemm_rcr_bias_sigmoid", "test_gemm_bias_sigmoid.py", [(64, 65)], 0, 0, True),
        ("gemm_rcr_bias_tanh", "test_gemm_bias_tanh.py", [(71, 71)], 0, 0, True),
        ("gemm_rcr_bias_swish", "test_gemm_bias_swish.py", [(36, 37), (68, 69)], 0, 0, True),
        ("gemm_rcr_bias_hardswish", "test_gemm_bias_hardswish.py", [(36, 37), (68, 69)], 0, 0, True),
        ("gemm_rcr_bias_mul_add", B, [(97, 101)], 1, 1, True),
        ("gemm_rcr_bias_sigmoid_mul", B, [(135, 140)], 1, 0, True),
        ("gemm_rcr_bias_sigmoid_mul_tanh", B, [(174, 179)], 1, 0, True),
        ("gemm_rcr_bias_add", B, [(216, 219)], 1, 0, True),
        ("gemm_rcr_bias_add_relu", B, [(253, 256)], 1, 0, True),
        ("gemm_rcr_bias_add_add_relu", B, [(290, 294)], 1, 1, True),
        ("gemm_rcr_bias_mul", B, [(336, 339)], 1, 0, True),
        ("gemm_rcr_bias_add_add", B, [(373, 377)], 1, 1, True),
        ("gemm_rcr_bias_mul_tanh", B, [(412, 415)], 1, 0, True),
    ]
    for case, fname, ranges, use_d0, use_d1, use_bias in gemm_cases:
        ns = {"torch": torch, "X_pt": x.float(), "W_pt": w.float(), "B_pt": b.float(),
              "D0_pt": d0.float(), "D1_pt": d1.float()}
        texts[case] = "".join(exec_reference_lines(ref_root, U + fname, lo, hi, ns) for lo, hi in ranges)
        ins = {"x": x, "w": w}
        if use_bias:
            ins["b"] = b
        if use_d0:
            ins["d0"] = d0
        if use_d1:
            ins["d1"] = d1
        put(case, ins, {"y": ns["Y_pt"]})

    # ---- gemm_rrr: test_gemm.py:220
    wr = rnd((40, 16), 25, 0.3)
    ns = {"torch": torch, "X_pt": x.float(), "W_pt": wr.float()}
    texts["gemm_rrr"] = exec_reference_lines(ref_root, U + "test_gemm.py", 220, 220, ns)
    put("gemm_rrr", {"x": x, "w": wr}, {"y": ns["Y_pt"]})

    # ---- gemm_rcr_bias_permute 20314: test_gemm_bias_permute.py:73-75
    m0, m1, n0, n1, n2 = 2, 8, 3, 4, 8  # shape=(t1, t2, t3) = (m1, n0, n1)
    xp, wp, bp = rnd((m0 * m1, 32), 5), rnd((n0 * n1 * n2, 32), 6), rnd((n0 * n1 * n2,), 7)
    ns = {"torch": torch, "X_pt": xp.float(), "W_pt": wp.float(), "B_pt": bp.float(),
          "M0": m0, "M1": m1, "N0": n0, "N1": n1, "N2": n2}
    texts["gemm_rcr_bias_permute"] = exec_reference_lines(ref_root, U + "test_gemm_bias_permute.py", 73, 75, ns)
    put("gemm_rcr_bias_permute", {"x": xp, "w": wp, "b": bp, "shape": torch.tensor([m1, n0, n1])}, {"y": ns["Y_pt"]})

    # ---- bmm_rcr: test_bmm.py:50-51
    xa, wa = rnd((3, 10, 24), 8), rnd((3, 12, 24), 9)
    ns = {"torch": torch, "X_pt": xa.float(), "W_pt": wa.float()}
    texts["bmm_rcr"] = exec_reference_lines(ref_root, U + "test_bmm.py", 50, 51, ns)
    put("bmm_rcr", {"a": xa, "b": wa}, {"y": ns["Y_pt"]})

    # ---- bmm_rrr: test_bmm.py:126; bmm_rrr_permute / bmm_rcr_permute: test_bmm_permute.py:55-57, 97-100
    wk = rnd((3, 24, 12), 26)
    ns = {"torch": torch, "X_pt": xa.float(), "W_pt": wk.float()}
    texts["bmm_rrr"] = exec_reference_lines(ref_root, U + "test_bmm.py", 126, 126, ns)
    put("bmm_rrr", {"a": xa, "b": wk}, {"y": ns["Y_pt"]})
    xb, wb_rrr, wb_rcr = rnd((6, 10, 24), 27), rnd((6, 24, 12), 28), rnd((6, 12, 24), 29)
    ns = {"torch": torch, "X_pt": xb.float(), "W_pt": wb_rrr.float(), "b": 6, "d1": 3, "m": 10, "N": 12}
    texts["bmm_rrr_permute"] = exec_reference_lines(ref_root, U + "test_bmm_permute.py", 55, 57, ns)
    put("bmm_rrr_permute", {"a": xb, "b": wb_rrr, "d1": torch.tensor([3])}, {"y": ns["Y_pt"]})
    ns = {"torch": torch, "X_pt": xb.float(), "W_pt": wb_rcr.float(), "b": 6, "d1": 3, "m": 10, "N": 12}
    texts["bmm_rcr_permute"] = exec_reference_lines(ref_root, U + "test_bmm_permute.py", 97, 100, ns)
    put("bmm_rcr_permute", {"a": xb, "b": wb_rcr, "d1": torch.tensor([3])}, {"y": ns["Y_pt"]})

    # ---- layernorm: test_layernorm.py:122
    x1, g1, b1 = rnd((6, 5, 48), 10), rnd((48,), 11), rnd((48,), 12)
    ns = {"torch": torch, "x1_pt": x1.float(), "x2_pt": g1.float(), "x3_pt": b1.float(), "NS": (48,), "eps": 1e-5}
    texts["layernorm"] = exec_reference_lines(ref_root, U + "test_layernorm.py", 122, 122, ns)
    put("layernorm", {"x": x1, "gamma": g1, "beta": b1}, {"y": ns["x4_pt"]})
    ns = {"torch": torch, "x1_pt": x1.float(), "x2_pt": None, "x3_pt": None, "NS": (5, 48), "eps": 1e-12}
    exec_reference_lines(ref_root, U + "test_layernorm.py", 122, 122, ns)
    put("layernorm_2d_no_affine", {"x": x1}, {"y": ns["x4_pt"]})

    # ---- softmax: test_softmax.py:85
    xs = rnd((4, 7, 33), 13, scale=2.0)
    for dim in (-1, 1):
        ns = {"torch": torch, "x_pt": xs.float(), "dim": dim}
        texts["softmax"] = exec_reference_lines(ref_root, U + "test_softmax.py", 85, 85, ns)
        put(f"softmax_dim{dim}", {"x": xs}, {"y": ns["y_pt"]})

    # ---- attention: the reference's functions, called
    ta = import_reference_attention_tests(ref_root)
    bsz, seq, heads, d = 2, 48, 3, 16
    qkv = rnd((bsz, seq, 3, heads, d), 14)
    mask = torch.ones(bsz, seq, dtype=torch.bool)
    for causal in (False, True):
        y = ta.attention_ref_math(qkv.float(), mask, 0.0, upcast=True, causal=causal)  # test_attention.py:111-139
        put(f"attention_ref_math_causal{int(causal)}", {"qkv": qkv}, {"y": y})
    # padded variable key lengths: the key mask of test_attention.py:519-523 (seq_range < lengths_kv) handed to the
    # same function, as the variable_seq_length_kv cases of that test do through attention_ref; a batch whose length
    # is 0 comes out NaN
    qkv3 = rnd((3, seq, 3, heads, d), 24)
    lengths_kv = torch.tensor([[seq], [17], [0]])
    key_mask = torch.arange(seq).unsqueeze(0).expand((3, seq)) < lengths_kv
    for causal in (False, True):
        y = ta.attention_ref_math(qkv3.float(), key_mask, 0.0, upcast=True, causal=causal)
        put(f"attention_ref_math_lengths_kv_causal{int(causal)}", {"qkv": qkv3, "lengths_kv": lengths_kv.reshape(-1)}, {"y": y})
    # attention_pt (test_attention.py:142-165): QKV projection, 20314 permute, attention; its scale is 64**-0.5
    nh, dd, sl = 2, 64, 40
    xq, wq, bq = rnd((sl, 32), 15), rnd((3 * nh * dd, 32), 16, 0.2), rnd((3 * nh * dd,), 17, 0.2)
    y = ta.attention_pt(xq.float(), wq.float(), bq.float(), nh, dd, sl)
    put("attention_pt", {"x": xq, "w": wq, "b": bq, "dims": torch.tensor([nh, dd, sl])}, {"y": y})
    # ref_cross_attention (test_attention.py:167-193), [B*H, S, D] operands with a shorter key length
    qc, kc, vc = rnd((6, 40, 24), 18), rnd((6, 13, 24), 19), rnd((6, 13, 24), 20)
    y = ta.ref_cross_attention(qc, kc, vc)
    put("ref_cross_attention", {"q": qc, "k": kc, "v": vc}, {"y": y})
    # ref_attention_bmhk (test_attention.py:182-193), [B, M, H, K] operands
    qb, kb, vb = rnd((2, 20, 3, 8), 21), rnd((2, 9, 3, 8), 22), rnd((2, 9, 3, 8), 23)
    y = ta.ref_cross_attention(qb, kb, vb)
    put("ref_attention_bmhk", {"q": qb, "k": kb, "v": vb}, {"y": y})

    path = os.path.join(HERE, "reference_numeric_fixtures.npz")
    np.savez_compressed(path, **out)
    for k, t in texts.items():  # shown, not stored: the reference's text stays in the reference
        print(f"[{k}] evaluated:\n{t}")
    print(f"wrote {len(out)} arrays, {os.path.getsize(path)} bytes, to {path}")


if __name__ == "__main__":
    main()
