"""GPU tests of the drop-in boundary: ops graph -> compile_model() -> Model.run_with_tensors().

Written the way the reference's tests are (tests/unittest/ops/test_gemm_rcr_bias_fast_gelu.py:72-100,
tests/unittest/backend/test_model_api.py): build a tiny graph, compile, run, compare with the oracle
expression; plus the runtime's error behaviour (wrong dtype / shape / count, dynamic-dim bounds,
closed model, unset constants).
"""
import os
import tempfile

import pytest
import torch

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu


def _imports():
    from aitemplate_b200.compiler import Model, compile_model, ops
    from aitemplate_b200.frontend import IntVar, Tensor, nn
    from aitemplate_b200.testing import detect_target

    return Model, compile_model, ops, IntVar, Tensor, nn, detect_target


def _rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).half()


def _close(got, want, tol=1e-2):
    got = got.float().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    err = (got - want).abs()
    assert bool((err <= tol + tol * want.abs()).all()), f"max abs err {float(err.max()):.4g}"


@pytest.fixture()
def workdir():
    with tempfile.TemporaryDirectory() as d:
        yield d


@pytest.mark.parametrize("ms", [[128], [1, 7, 64, 127]])
def test_gemm_rcr_bias_fast_gelu_static_and_dynamic_m(workdir, ms):
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    from aitemplate_b200.utils import shape_utils

    k, n = 1024, 64
    m_dim = shape_utils.gen_int_var_min_max(ms, name="m")
    X = Tensor(shape=[m_dim, k], dtype="float16", name="input_0", is_input=True)
    W = Tensor(shape=[n, k], dtype="float16", name="input_1", is_input=True)
    B = Tensor(shape=[n], dtype="float16", name="input_2", is_input=True)
    Y = ops.gemm_rcr_bias_fast_gelu()(X, W, B)
    Y._attrs["name"] = "output_0"
    Y._attrs["is_output"] = True
    module = compile_model(Y, detect_target(), workdir, f"gemm_rcr_bias_fast_gelu_{len(ms)}")
    for m in ms:
        x, w, b = _rand((m, k), 1), _rand((n, k), 2, 0.05), _rand((n,), 3)
        y = torch.empty((max(ms), n), dtype=torch.float16, device="cuda")
        res = module.run_with_tensors({"input_0": x.cuda(), "input_1": w.cuda(), "input_2": b.cuda()}, [y])
        assert tuple(res["output_0"].shape) == (m, n)
        _close(res["output_0"], oracle.gemm_rcr(x, w, b, epilogue="fast_gelu"))


def test_dynamic_dim_out_of_range_is_an_error(workdir):
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    X = Tensor(shape=[IntVar([2, 16], name="m"), 64], name="x", is_input=True)
    W = Tensor(shape=[32, 64], name="w", is_input=True)
    Y = ops.gemm_rcr()(X, W)
    Y._attrs["name"] = "y"
    Y._attrs["is_output"] = True
    module = compile_model(Y, detect_target(), workdir, "dyn_bounds")
    w = _rand((32, 64), 1).cuda()
    y = torch.empty((16, 32), dtype=torch.float16, device="cuda")
    for bad_m in (1, 17):
        with pytest.raises(RuntimeError, match="AITemplateModelContainerRun"):
            module.run_with_tensors([_rand((bad_m, 64), 2).cuda(), w], [y])
    ok = module.run_with_tensors([_rand((5, 64), 2).cuda(), w], [y])
    assert tuple(ok["y"].shape) == (5, 32)


def test_runtime_argument_errors(workdir):
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    X = Tensor(shape=[8, 64], name="x", is_input=True)
    W = Tensor(shape=[32, 64], name="w", is_input=True)
    Y = ops.gemm_rcr()(X, W)
    Y._attrs["name"] = "y"
    Y._attrs["is_output"] = True
    module = compile_model(Y, detect_target(), workdir, "arg_errors")
    x, w = _rand((8, 64), 1).cuda(), _rand((32, 64), 2).cuda()
    y = torch.empty((8, 32), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):  # CPU tensor
        module.run_with_tensors([x.cpu(), w], [y])
    with pytest.raises(ValueError):  # non-contiguous
        module.run_with_tensors([x.t().contiguous().t(), w], [y])
    with pytest.raises(ValueError):  # unknown input name
        module.run_with_tensors({"x": x, "nope": w}, [y])
    with pytest.raises(ValueError):  # wrong count in a dict
        module.run_with_tensors({"x": x}, [y])
    with pytest.raises(RuntimeError):  # wrong count in a list
        module.run_with_tensors([x], [y])
    with pytest.raises(RuntimeError):  # wrong dtype
        module.run_with_tensors([x.float(), w], [y])
    with pytest.raises(RuntimeError):  # wrong static shape
        module.run_with_tensors([_rand((8, 32), 1).cuda(), w], [y])
    assert module.get_input_name_to_index_map() == {"x": 0, "w": 1}
    assert module.get_output_name_to_index_map() == {"y": 0}
    assert module.get_output_maximum_shape(0) == [8, 32]
    assert module.get_output_dtype(0) == 1
    assert module.get_num_runtimes() == 1
    module.close()
    with pytest.raises(RuntimeError, match="closed"):
        module.run_with_tensors([x, w], [y])


def test_constants_bound_unbound_and_double_buffer(workdir):
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    X = Tensor(shape=[16, 64], name="x", is_input=True)
    W = Tensor(shape=[32, 64], name="w")
    B = Tensor(shape=[32], name="b")
    Y = ops.gemm_rcr_bias()(X, W, B)
    Y._attrs["name"] = "y"
    Y._attrs["is_output"] = True
    w, b, x = _rand((32, 64), 1, 0.1), _rand((32,), 2), _rand((16, 64), 3)
    module = compile_model(Y, detect_target(), workdir, "constants", constants={"w": w})
    y = torch.empty((16, 32), dtype=torch.float16, device="cuda")
    assert sorted(module.get_constant_names(unbound_constants_only=False)) == ["b", "w"]
    assert module.get_constant_names() == ["b"]
    with pytest.raises(RuntimeError, match="Run"):  # b was never set
        module.run_with_tensors([x.cuda()], [y])
    module.set_constant_with_tensor("b", b.cuda())
    _close(module.run_with_tensors([x.cuda()], [y])["y"], oracle.gemm_rcr(x, w, b))
    with pytest.raises(RuntimeError):  # wrong size
        module.set_constant_with_tensor("b", _rand((31,), 4).cuda())
    with pytest.raises(RuntimeError):  # unknown name
        module.set_constant_with_tensor("nope", b.cuda())
    # double buffering: the new value is only used after swap_constants()
    w2 = _rand((32, 64), 5, 0.1)
    module.set_double_buffer_constant_with_tensor("w", w2.cuda())
    _close(module.run_with_tensors([x.cuda()], [y])["y"], oracle.gemm_rcr(x, w, b))
    module.swap_constants()
    _close(module.run_with_tensors([x.cuda()], [y])["y"], oracle.gemm_rcr(x, w2, b))
    # AIT_RECOMPILE=0 reloads the stored plan (bound constants included)
    os.environ["AIT_RECOMPILE"] = "0"
    try:
        again = compile_model(Y, detect_target(), workdir, "constants")
    finally:
        del os.environ["AIT_RECOMPILE"]
    again.set_constant_with_tensor("b", b.cuda())
    _close(again.run_with_tensors([x.cuda()], [y])["y"], oracle.gemm_rcr(x, w, b))


def test_fuse_mm_elementwise_and_views(workdir):
    """gemm_rcr + ADD(bias) + FASTGELU written with plain ops is fused into one launch, and an
    output that is a view of an intermediate is written in place."""
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    from aitemplate_b200.compiler.ops import FuncEnum

    batch = IntVar([1, 8], name="batch")
    X = Tensor(shape=[batch, 48, 64], name="x", is_input=True)
    W = Tensor(shape=[96, 64], name="w", is_input=True)
    B = Tensor(shape=[96], name="b", is_input=True)
    h = ops.gemm_rcr()(ops.reshape()(X, [-1, 64]), W)
    h = ops.elementwise(FuncEnum.FASTGELU)(ops.elementwise(FuncEnum.ADD)(h, B))
    Y = ops.reshape()(h, [batch, 48, 96])
    Y._attrs["name"] = "y"
    Y._attrs["is_output"] = True
    module = compile_model(Y, detect_target(), workdir, "fuse")
    kernels = [op._attrs["op"] for t in module.debug_sorted_graph for op in t._attrs["src_ops"]]
    assert "gemm_rcr_bias_fast_gelu" in kernels and "elementwise" not in kernels
    for bsz in (1, 3, 8):
        x, w, b = _rand((bsz, 48, 64), 1), _rand((96, 64), 2, 0.1), _rand((96,), 3)
        y = torch.empty((8, 48, 96), dtype=torch.float16, device="cuda")
        res = module.run_with_tensors({"x": x.cuda(), "w": w.cuda(), "b": b.cuda()}, {"y": y})
        assert tuple(res["y"].shape) == (bsz, 48, 96)
        _close(res["y"], oracle.gemm_rcr(x, w, b, epilogue="fast_gelu"))


def test_layout_ops_in_a_graph_are_bit_exact(workdir):
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    xs = [Tensor(shape=[64, 32 * (i + 1)], name=f"x{i}", is_input=True) for i in range(3)]
    cat = ops.concatenate()(xs, dim=1)
    a, b = ops.split()(cat, [64, 128], dim=1)
    p = ops.permute()(ops.reshape()(b, [64, 4, 32]), [1, 0, 2])
    outs = []
    for name, t in (("cat", cat), ("a", a), ("p", p)):
        t._attrs["name"] = name
        t._attrs["is_output"] = True
        outs.append(t)
    module = compile_model(outs, detect_target(), workdir, "layout")
    data = [_rand((64, 32 * (i + 1)), i) for i in range(3)]
    bufs = {"cat": torch.empty((64, 192), dtype=torch.float16, device="cuda"),
            "a": torch.empty((64, 64), dtype=torch.float16, device="cuda"),
            "p": torch.empty((4, 64, 32), dtype=torch.float16, device="cuda")}
    res = module.run_with_tensors({f"x{i}": d.cuda() for i, d in enumerate(data)}, bufs)
    want = torch.cat(data, 1)
    assert torch.equal(res["cat"].cpu(), want)
    assert torch.equal(res["a"].cpu(), want[:, :64])
    assert torch.equal(res["p"].cpu(), want[:, 64:].reshape(64, 4, 32).permute(1, 0, 2).contiguous())


def test_softmax_layernorm_bmm_attention_graph(workdir):
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    q = Tensor(shape=[2, 4, 96, 64], name="q", is_input=True)
    k = Tensor(shape=[2, 4, 80, 64], name="k", is_input=True)
    v = Tensor(shape=[2, 4, 80, 64], name="v", is_input=True)
    att = ops.mem_eff_attention(causal=False)(q, k, v)
    att._attrs["name"] = "att"
    att._attrs["is_output"] = True
    s = ops.bmm_rcr()(ops.reshape()(q, [8, 96, 64]), ops.reshape()(k, [8, 80, 64]))
    sm = ops.softmax()(s, -1)
    sm._attrs["name"] = "sm"
    sm._attrs["is_output"] = True
    ln = ops.layernorm()(ops.reshape()(att, [2 * 96, 256]), None, None, [256], 1e-5)
    ln._attrs["name"] = "ln"
    ln._attrs["is_output"] = True
    module = compile_model([att, sm, ln], detect_target(), workdir, "mixed")
    qd, kd, vd = _rand((2, 4, 96, 64), 1), _rand((2, 4, 80, 64), 2), _rand((2, 4, 80, 64), 3)
    bufs = {"att": torch.empty((2, 96, 4, 64), dtype=torch.float16, device="cuda"),
            "sm": torch.empty((8, 96, 80), dtype=torch.float16, device="cuda"),
            "ln": torch.empty((192, 256), dtype=torch.float16, device="cuda")}
    res = module.run_with_tensors({"q": qd.cuda(), "k": kd.cuda(), "v": vd.cuda()}, bufs)
    want_att = oracle.mem_eff_attention(qd, kd, vd)
    _close(res["att"], want_att, 4e-3)
    want_s = oracle.bmm_rcr(qd.reshape(8, 96, 64), kd.reshape(8, 80, 64))
    _close(res["sm"], oracle.softmax(want_s.half(), -1), 1e-2)
    _close(res["ln"], oracle.layernorm(res["att"].reshape(192, 256).cpu(), None, None), 4e-3)


@pytest.mark.parametrize("graph_mode", [False, True])
def test_bert_layer_matches_oracle(workdir, graph_mode):
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    from aitemplate_b200.testing import workloads

    batch, seq = 4, 384
    x, params = workloads.bert_layer_inputs(batch, seq)
    _, y = workloads.build_bert_layer(batch, seq)
    module = compile_model(y, detect_target(), workdir, "bert_layer", num_runtimes=2)
    module.set_many_constants_with_tensors({n: params[k].cuda() for n, k in workloads.BERT_PARAM_NAMES.items()})
    out = torch.empty((batch, seq, 768), dtype=torch.float16, device="cuda")
    want = oracle.bert_layer(x, params)
    for _ in range(3):  # eager warm-up, capture, replay
        out.zero_()
        res = module.run_with_tensors({"hidden_states": x.cuda()}, {"output_0": out}, graph_mode=graph_mode)
        _close(res["output_0"], want, 2e-2)
    mean, std, _ = module.benchmark_with_tensors({"hidden_states": x.cuda()}, {"output_0": out}, count=5, repeat=2,
                                                 graph_mode=graph_mode)
    assert mean > 0
    prof = os.path.join(workdir, "prof.json")
    module.profile_with_tensors({"hidden_states": x.cuda()}, {"output_0": out}, 2, prof)
    import json

    with open(prof) as f:
        names = list(json.load(f).keys())
    assert sum(n.startswith("gemm_rcr") for n in names) == 4 and any(n.startswith("mem_eff_attention") for n in names)


@pytest.mark.parametrize("tokens", [1024, 4096])
def test_sd_transformer_block_matches_oracle(workdir, tokens):
    # benchmark configuration 3: Stable-Diffusion UNet transformer block, batch 2, dim 320, 8 heads x 40
    # (head dim 40 = 5 x 8: the tensor-core attention path with a zero-padded head), self-attention over the
    # latent tokens, cross-attention against 77 context tokens of dim 768, GEGLU feed-forward.
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    from aitemplate_b200.testing import workloads

    batch = 2
    x, context, params = workloads.sd_block_inputs(batch, tokens)
    y = workloads.build_sd_block(batch, tokens=tokens)
    module = compile_model(y, detect_target(), workdir, "sd_block")
    module.set_many_constants_with_tensors({k: v.cuda() for k, v in params.items()})
    out = torch.empty((batch, tokens, 320), dtype=torch.float16, device="cuda")
    want = oracle.sd_transformer_block(x, context, params)
    for graph_mode in (False, True, True):
        out.zero_()
        res = module.run_with_tensors({"latent": x.cuda(), "context": context.cuda()}, {"output_0": out},
                                      graph_mode=graph_mode)
        _close(res["output_0"], want, 2e-2)


@pytest.mark.parametrize("m", [64, 1000])
def test_strided_output_fusion_into_concat(workdir, m):
    # GEMMs and a layernorm write their column blocks straight into the concatenated buffer
    # (tests/unittest/compiler/test_strided_op_cat_pattern.py, test_strided_layernorm.py); widths chosen so that
    # one block starts 16-byte aligned (vector / TMA store) and one does not (scalar store path)
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    from aitemplate_b200.frontend import IntImm

    kdim = 128
    x = Tensor([m, kdim], name="x", is_input=True)
    z = Tensor([m, 20], name="z", is_input=True)
    w1, b1 = Tensor([96, kdim], name="w1"), Tensor([96], name="b1")
    w2 = Tensor([264, kdim], name="w2")
    g1 = ops.gemm_rcr_bias_relu()(x, w1, b1)
    g2 = ops.gemm_rcr()(x, w2)
    ln = ops.layernorm()(x, None, None, [IntImm(kdim)], 1e-5)
    y = ops.concatenate()([g1, z, g2, ln], dim=1)
    y._attrs["name"], y._attrs["is_output"] = "y", True
    module = compile_model(y, detect_target(), workdir, "strided_cat")
    plan = open(os.path.join(workdir, "strided_cat", "test.so.plan")).read()
    assert [l for l in plan.splitlines() if l.startswith("op concatenate")][0].split()[-7:-1] == ["1", "4", "0", "1", "0", "0"]
    xd, zd = _rand((m, kdim), 1), _rand((m, 20), 2)
    w1d, b1d, w2d = _rand((96, kdim), 3, 0.05), _rand((96,), 4, 0.1), _rand((264, kdim), 5, 0.05)
    module.set_many_constants_with_tensors({"w1": w1d.cuda(), "b1": b1d.cuda(), "w2": w2d.cuda()})
    out = torch.full((m, 96 + 20 + 264 + kdim), 9.0, dtype=torch.float16, device="cuda")
    res = module.run_with_tensors({"x": xd.cuda(), "z": zd.cuda()}, {"y": out})["y"]
    want = torch.cat([oracle.gemm_rcr(xd, w1d, b1d, epilogue="relu"), zd.float(), oracle.gemm_rcr(xd, w2d),
                      oracle.layernorm(xd, None, None)], dim=1)
    _close(res, want, 1e-2)
    assert torch.equal(res[:, 96:116].cpu(), zd)  # the copied block is bit-exact


@pytest.mark.parametrize("m", [48, 1000])
def test_strided_input_fusion_from_split(workdir, m):
    # GEMMs (operand A) and layernorms read their column blocks of a last-dim split's input in place
    # (tests/unittest/compiler/test_split_bmm_fusion.py, test_strided_layernorm.py in the reference); the block with
    # an elementwise reader is still copied by the split kernel
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    from aitemplate_b200.compiler.ops import FuncEnum
    from aitemplate_b200.frontend import IntImm

    widths = [256, 64, 32, 72]
    x = Tensor([m, sum(widths)], name="x", is_input=True)
    w1, b1 = Tensor([136, 256], name="w1"), Tensor([136], name="b1")
    w2 = Tensor([264, 64], name="w2")
    p0, p1, p2, p3 = ops.split()(x, widths, dim=-1)
    outs = {
        "g1": ops.gemm_rcr_bias_relu()(p0, w1, b1),
        "ln0": ops.layernorm()(p0, None, None, [IntImm(256)], 1e-5),
        "g2": ops.gemm_rcr()(p1, w2),
        "e2": ops.elementwise(FuncEnum.RELU)(p2),
        "ln3": ops.layernorm()(p3, None, None, [IntImm(72)], 1e-5),
    }
    for name, t in outs.items():
        t._attrs["name"], t._attrs["is_output"] = name, True
    module = compile_model(list(outs.values()), detect_target(), workdir, "strided_split")
    plan = open(os.path.join(workdir, "strided_split", "test.so.plan")).read()
    split_line = next(l for l in plan.splitlines() if l.startswith("op split")).split()
    assert split_line[-5:-1] == ["0", "0", "1", "0"]
    xd = _rand((m, sum(widths)), 1)
    w1d, b1d, w2d = _rand((136, 256), 3, 0.05), _rand((136,), 4, 0.1), _rand((264, 64), 5, 0.05)
    module.set_many_constants_with_tensors({"w1": w1d.cuda(), "b1": b1d.cuda(), "w2": w2d.cuda()})
    bufs = {"g1": (m, 136), "ln0": (m, 256), "g2": (m, 264), "e2": (m, 32), "ln3": (m, 72)}
    res = module.run_with_tensors(
        {"x": xd.cuda()}, {k: torch.full(v, 9.0, dtype=torch.float16, device="cuda") for k, v in bufs.items()})
    c0, c1, c2, c3 = torch.split(xd, widths, dim=1)
    _close(res["g1"], oracle.gemm_rcr(c0, w1d, b1d, epilogue="relu"), 1e-2)
    _close(res["ln0"], oracle.layernorm(c0, None, None), 1e-2)
    _close(res["g2"], oracle.gemm_rcr(c1, w2d), 1e-2)
    assert torch.equal(res["e2"].cpu(), torch.relu(c2))
    _close(res["ln3"], oracle.layernorm(c3, None, None), 1e-2)


def test_mem_eff_attention_with_lengths_in_a_graph(workdir):
    # tests/unittest/ops/test_attention.py:456-742 with variable_seq_length_kv / variable_seq_length_q: int32 lengths
    # tensors as graph inputs
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    b, h, s, d = 5, 4, 192, 64
    q = Tensor([b, h, s, d], name="q", is_input=True)
    k = Tensor([b, h, s, d], name="k", is_input=True)
    v = Tensor([b, h, s, d], name="v", is_input=True)
    lkv = Tensor([b, 1], name="lengths_kv", dtype="int", is_input=True)
    lq = Tensor([b, 1], name="lengths_q", dtype="int", is_input=True)
    y = ops.mem_eff_attention(causal=False, variable_seq_length_kv=True, variable_seq_length_q=True)(q, k, v, lkv, lq)
    y._attrs["name"], y._attrs["is_output"] = "output", True
    module = compile_model(y, detect_target(), workdir, "attention_lengths")
    qd, kd, vd = _rand((b, h, s, d), 1), _rand((b, h, s, d), 2), _rand((b, h, s, d), 3)
    lengths_kv = torch.tensor([192, 7, 0, 64, 100], dtype=torch.int32)
    lengths_q = torch.tensor([192, 192, 50, 0, 129], dtype=torch.int32)
    out = torch.full((b, s, h, d), 5.0, dtype=torch.float16, device="cuda")
    res = module.run_with_tensors({"q": qd.cuda(), "k": kd.cuda(), "v": vd.cuda(),
                                   "lengths_kv": lengths_kv.reshape(b, 1).cuda(),
                                   "lengths_q": lengths_q.reshape(b, 1).cuda()}, {"output": out})
    got = res["output"].float().cpu()
    want = oracle.mem_eff_attention(qd, kd, vd, lengths_kv=lengths_kv, lengths_q=lengths_q)
    for i in range(b):
        rows = int(lengths_q[i])
        assert bool((got[i, rows:] == 5.0).all())
        if int(lengths_kv[i]) == 0:
            assert bool(torch.isnan(got[i, :rows]).all())
        else:
            _close(got[i, :rows], want[i, :rows], 1e-2)


def test_strided_operand_b_from_split(workdir):
    # gemm_rcr reads operand B ([N, K]) in place from a block of K columns of a wider tensor: no split kernel runs
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    from aitemplate_b200 import _lib

    n, k0, k1, m = 136, 256, 64, 40
    wide = Tensor([n, k0 + k1], name="wide", is_input=True)
    x0, x1 = Tensor([m, k0], name="x0", is_input=True), Tensor([m, k1], name="x1", is_input=True)
    bias = Tensor([n], name="bias")
    w0, w1 = ops.split()(wide, [k0, k1], dim=-1)
    outs = {"y0": ops.gemm_rcr_bias_relu()(x0, w0, bias), "y1": ops.gemm_rcr()(x1, w1)}
    for name, t in outs.items():
        t._attrs["name"], t._attrs["is_output"] = name, True
    module = compile_model(list(outs.values()), detect_target(), workdir, "strided_b")
    wd, x0d, x1d, bd = _rand((n, k0 + k1), 1, 0.05), _rand((m, k0), 2), _rand((m, k1), 3), _rand((n,), 4, 0.1)
    module.set_many_constants_with_tensors({"bias": bd.cuda()})
    ins = {"wide": wd.cuda(), "x0": x0d.cuda(), "x1": x1d.cuda()}
    bufs = {name: torch.full((m, n), 9.0, dtype=torch.float16, device="cuda") for name in outs}
    launches = _lib.kernel_launch_count()
    res = module.run_with_tensors(ins, bufs)
    assert _lib.kernel_launch_count() - launches == 2  # the two GEMMs: the split launches nothing
    _close(res["y0"], oracle.gemm_rcr(x0d, wd[:, :k0], bd, epilogue="relu"), 1e-2)
    _close(res["y1"], oracle.gemm_rcr(x1d, wd[:, k0:]), 1e-2)


def test_bmm_permute_ops_in_a_graph(workdir):
    # bmm_rcr_permute / bmm_rrr_permute (tests/unittest/ops/test_bmm_permute.py): the 0213 permutation is fused into
    # the batched GEMM's store and the node returns the [B / d1, M, d1, N] view
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    bsz, m, n, kk, d1 = 24, 80, 64, 88, 12
    a = Tensor([bsz, m, kk], name="a", is_input=True)
    b = Tensor([bsz, n, kk], name="b", is_input=True)
    c = Tensor([bsz, kk, n], name="c", is_input=True)
    y0 = ops.bmm_rcr_permute(shape=(d1,))(a, b)
    op1 = ops.bmm_rrr_permute(shape=(d1,))
    y1 = ops.bmm_rrr_permute(**op1._get_op_attributes())(a, c)
    for name, t in (("y0", y0), ("y1", y1)):
        t._attrs["name"], t._attrs["is_output"] = name, True
    assert [d.value() for d in y0._attrs["shape"]] == [bsz // d1, m, d1, n]
    module = compile_model([y0, y1], detect_target(), workdir, "bmm_permute")
    ad, bd, cd = _rand((bsz, m, kk), 1), _rand((bsz, n, kk), 2), _rand((bsz, kk, n), 3)
    outs = {k: torch.empty((bsz // d1, m, d1, n), dtype=torch.float16, device="cuda") for k in ("y0", "y1")}
    res = module.run_with_tensors({"a": ad.cuda(), "b": bd.cuda(), "c": cd.cuda()}, outs)
    _close(res["y0"], oracle.bmm_permute(ad, bd, d1), 1e-2)
    _close(res["y1"], oracle.bmm_permute(ad, cd, d1, b_row_major=True), 1e-2)


def test_gemm_permute0213_fusion_matches_oracle(workdir):
    # q-projection -> [B, S, H, d] -> heads first: the permute is folded into the GEMM's staged store
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    bsz, seq, heads, d, kdim = 3, 160, 4, 64, 192
    x = Tensor([bsz * seq, kdim], name="x", is_input=True)
    w, b = Tensor([heads * d, kdim], name="w"), Tensor([heads * d], name="b")
    y = ops.permute()(ops.reshape()(ops.gemm_rcr_bias()(x, w, b), [bsz, seq, heads, d]), [0, 2, 1, 3])
    y._attrs["name"], y._attrs["is_output"] = "y", True
    module = compile_model(y, detect_target(), workdir, "gemm_permute0213")
    plan = open(os.path.join(workdir, "gemm_permute0213", "test.so.plan")).read()
    assert "op permute" not in plan
    xd, wd, bd = _rand((bsz * seq, kdim), 1), _rand((heads * d, kdim), 2, 0.05), _rand((heads * d,), 3, 0.1)
    module.set_many_constants_with_tensors({"w": wd.cuda(), "b": bd.cuda()})
    out = torch.empty((bsz, heads, seq, d), dtype=torch.float16, device="cuda")
    res = module.run_with_tensors({"x": xd.cuda()}, {"y": out})["y"]
    want = oracle.gemm_rcr(xd, wd, bd).reshape(bsz, seq, heads, d).permute(0, 2, 1, 3)
    _close(res, want, 1e-2)


@pytest.mark.parametrize("bsz,m", [(4, 96), (3, 300)])
def test_bmm_reads_split_blocks_and_writes_concat_blocks(workdir, bsz, m):
    # tests/unittest/compiler/test_split_bmm_fusion.py, test_strided_op_cat_pattern.py in the reference: both bmm
    # operands are column blocks of last-dim splits and both results are column blocks of one concatenate
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    k1, k2, n1, n2 = 64, 136, 72, 264
    x = Tensor([bsz, m, k1 + k2], name="x", is_input=True)
    w = Tensor([bsz, n1, k1 + k2], name="w", is_input=True)
    v = Tensor([bsz, k2, n2], name="v", is_input=True)
    xa, xb = ops.split()(x, [k1, k2], dim=2)
    wa, wb = ops.split()(w, [k1, k2], dim=2)
    y = ops.concatenate()([ops.bmm_rcr()(xa, wa), ops.bmm_rrr()(xb, v), ops.bmm_rcr()(xb, wb)], dim=2)
    y._attrs["name"], y._attrs["is_output"] = "y", True
    module = compile_model(y, detect_target(), workdir, "bmm_strided")
    plan = open(os.path.join(workdir, "bmm_strided", "test.so.plan")).read()
    assert [l.split()[-4:-1] for l in plan.splitlines() if l.startswith("op concatenate")] == [["0", "0", "0"]]
    assert all(l.split()[-3:-1] == ["0", "0"] for l in plan.splitlines() if l.startswith("op split"))
    xd, wd, vd = _rand((bsz, m, k1 + k2), 1), _rand((bsz, n1, k1 + k2), 2, 0.1), _rand((bsz, k2, n2), 3, 0.1)
    out = torch.full((bsz, m, n1 + n2 + n1), 9.0, dtype=torch.float16, device="cuda")
    res = module.run_with_tensors({"x": xd.cuda(), "w": wd.cuda(), "v": vd.cuda()}, {"y": out})["y"]
    want = torch.cat([oracle.bmm_rcr(xd[:, :, :k1], wd[:, :, :k1]), oracle.bmm_rrr(xd[:, :, k1:], vd),
                      oracle.bmm_rcr(xd[:, :, k1:], wd[:, :, k1:])], dim=2)
    _close(res, want, 1e-2)


def test_compile_time_gemm_profiling(workdir):
    # profile_devs given: every GEMM of the graph is timed over the launch configurations, the winners go into the
    # plan and a cache file, and the model still matches the oracle
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    from aitemplate_b200.backend.profiler_cache import GemmProfileCache

    m, k, n = 512, 1024, 768
    x = Tensor([m, k], name="x", is_input=True)
    w, b = Tensor([n, k], name="w"), Tensor([n], name="b")
    y = ops.gemm_rcr_bias_fast_gelu()(x, w, b)
    y._attrs["name"], y._attrs["is_output"] = "y", True
    module = compile_model(y, detect_target(), workdir, "profiled", profile_devs=[0], profile_dir=workdir)
    cache = GemmProfileCache(os.path.join(workdir, "gemm_profile_cache.json"))
    assert len(cache.entries) == 1
    (entry,) = cache.entries.values()
    assert entry["tile_n"] in (0, 64, 128, 256, 512) and entry["us"] > 0
    plan = open(os.path.join(workdir, "profiled", "test.so.plan")).read()
    gemm_line = next(l for l in plan.splitlines() if l.startswith("op gemm_rcr")).split()
    assert str(entry["tile_n"]) in gemm_line and plan.count("op gemm_rcr") == 1
    xd, wd, bd = _rand((m, k), 1), _rand((n, k), 2, 0.02), _rand((n,), 3, 0.02)
    module.set_many_constants_with_tensors({"w": wd.cuda(), "b": bd.cuda()})
    out = torch.empty((m, n), dtype=torch.float16, device="cuda")
    res = module.run_with_tensors({"x": xd.cuda()}, {"y": out})["y"]
    _close(res, oracle.gemm_rcr(xd, wd, bd, epilogue="fast_gelu"), 1e-2)


def test_row_major_b_ops_in_a_graph(workdir):
    # gemm_rrr_bias -> bmm_rrr (the unfused attention form P @ V uses bmm_rrr in the reference's examples)
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()

    x = Tensor([IntVar([1, 256], name="m"), 96], name="x", is_input=True)
    w, b = Tensor([96, 160], name="w"), Tensor([160], name="b")
    p_ = Tensor([4, 48, 40], name="p", is_input=True)
    v = Tensor([4, 40, 24], name="v", is_input=True)
    y = ops.gemm_rrr_bias()(x, w, b)
    y._attrs["name"], y._attrs["is_output"] = "y", True
    z = ops.bmm_rrr()(p_, v)
    z._attrs["name"], z._attrs["is_output"] = "z", True
    module = compile_model([y, z], detect_target(), workdir, "rrr")
    wd, bd = _rand((96, 160), 1, 0.1), _rand((160,), 2, 0.1)
    module.set_many_constants_with_tensors({"w": wd.cuda(), "b": bd.cuda()})
    pd, vd = _rand((4, 48, 40), 3), _rand((4, 40, 24), 4)
    for m in (1, 77, 256):
        xd = _rand((m, 96), 5 + m)
        outs = {"y": torch.empty((m, 160), dtype=torch.float16, device="cuda"),
                "z": torch.empty((4, 48, 24), dtype=torch.float16, device="cuda")}
        res = module.run_with_tensors({"x": xd.cuda(), "p": pd.cuda(), "v": vd.cuda()}, outs)
        _close(res["y"], oracle.gemm_rrr(xd, wd, bd))
        _close(res["z"], oracle.bmm_rrr(pd, vd), 2e-2)


def test_concurrent_runs_share_the_pool(workdir):
    import threading

    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    X = Tensor(shape=[256, 128], name="x", is_input=True)
    W = Tensor(shape=[128, 128], name="w", is_input=True)
    Y = ops.gemm_rcr()(ops.gemm_rcr()(X, W), W)
    Y._attrs["name"] = "y"
    Y._attrs["is_output"] = True
    module = compile_model(Y, detect_target(), workdir, "pool", num_runtimes=2)
    x, w = _rand((256, 128), 1), _rand((128, 128), 2, 0.1)
    want = oracle.gemm_rcr(oracle.gemm_rcr(x, w).half(), w)
    xg, wg = x.cuda(), w.cuda()
    results, errors = [None] * 4, []

    def worker(i):
        try:
            torch.cuda.set_device(0)
            s = torch.cuda.Stream()
            y = torch.empty((256, 128), dtype=torch.float16, device="cuda")
            with torch.cuda.stream(s):
                for _ in range(10):
                    module.run_with_tensors([xg, wg], [y], stream_ptr=s.cuda_stream, sync=True)
            results[i] = y
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for y in results:
        _close(y, want, 2e-2)


def test_multihead_attention_default_flash_path_matches_oracle(workdir):
    """nn.MultiheadAttention as the reference's BERT example uses it (examples/03_bert/modeling/bert.py:55-66): the
    packed flash_attention path with the cu_length constant, written with `aitemplate.*` imports only."""
    from aitemplate.compiler import compile_model
    from aitemplate.frontend import nn, Tensor
    from aitemplate.testing import detect_target

    batch, seq, hidden, heads = 3, 384, 768, 12
    attn = nn.MultiheadAttention(dim=hidden, batch_size=batch, seq_len=seq, num_heads=heads, qkv_bias=True,
                                 has_residual=True)
    attn.name_parameter_tensor()
    x = Tensor([batch, seq, hidden], name="hidden_states", is_input=True)
    y = attn(x, x)
    y._attrs["name"], y._attrs["is_output"] = "output_0", True
    module = compile_model(y, detect_target(), workdir, "mha_flash")
    g = torch.Generator().manual_seed(77)
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).half()  # noqa: E731
    p = {"qkv_weight": r(3 * hidden, hidden, sc=0.02), "qkv_bias": r(3 * hidden, sc=0.02),
         "proj_weight": r(hidden, hidden, sc=0.02), "proj_bias": r(hidden, sc=0.02)}
    xh = r(batch, seq, hidden)
    cu = torch.arange(batch + 1, dtype=torch.int32) * seq
    module.set_many_constants_with_tensors({**{k: v.cuda() for k, v in p.items()}, "cu_length": cu.cuda()})
    out = torch.empty((batch, seq, hidden), dtype=torch.float16, device="cuda")
    x2 = xh.float().reshape(batch * seq, hidden)
    qkv = oracle.gemm_rcr_bias_permute(x2, p["qkv_weight"], p["qkv_bias"], (seq, 3, heads), "20314")
    a = oracle.mem_eff_attention(qkv[0], qkv[1], qkv[2]).reshape(batch * seq, hidden)
    want = oracle.gemm_rcr(a.half(), p["proj_weight"], p["proj_bias"], x2, epilogue="add").reshape(batch, seq, hidden)
    for graph_mode in (False, True, True):
        res = module.run_with_tensors({"hidden_states": xh.cuda()}, {"output_0": out}, graph_mode=graph_mode)
        _close(res["output_0"], want, 2e-2)
    module.close()


def test_dynamic_m_reserves_split_k_workspace_for_interior_sizes(workdir):
    """Split-K demand is not monotonic in M (nothing at M = 1, nothing once the tiles fill the SMs, most in
    between), so a dynamic M in [1, 4096] must reserve scratch for the interior sizes, not only for its bounds;
    otherwise M = 256 silently runs unsplit."""
    import ctypes

    from aitemplate_b200 import kernels
    from aitemplate_b200.compiler import AITemplateAllocatorKind

    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    k, n = 8192, 1024
    need = kernels.gemm_workspace_bytes(1, 256, n, k)
    assert need > 0, "M = 256 is meant to split K"
    assert kernels.gemm_workspace_bytes(1, 4096, n, k) == 0 or kernels.gemm_workspace_bytes(1, 4096, n, k) < need
    X = Tensor(shape=[IntVar([1, 4096], name="m"), k], dtype="float16", name="input_0", is_input=True)
    W = Tensor(shape=[n, k], dtype="float16", name="input_1", is_input=True)
    B = Tensor(shape=[n], dtype="float16", name="input_2", is_input=True)
    Y = ops.gemm_rcr_bias_relu()(X, W, B)
    Y._attrs["name"], Y._attrs["is_output"] = "output_0", True
    module = compile_model(Y, detect_target(), workdir, "dyn_m_workspace", allocator_kind=AITemplateAllocatorKind.TRACKING)
    nbytes = ctypes.c_size_t(0)
    module.DLL.AITemplateTrackingAllocatorGetNumBytes(module.allocator_handle, ctypes.byref(nbytes))
    assert nbytes.value >= need, (nbytes.value, need)
    w, b = _rand((n, k), 2, 0.02), _rand((n,), 3)
    for m in (1, 256, 300, 4096):
        x = _rand((m, k), 10 + m)
        y = torch.empty((4096, n), dtype=torch.float16, device="cuda")
        res = module.run_with_tensors({"input_0": x.cuda(), "input_1": w.cuda(), "input_2": b.cuda()}, [y])
        _close(res["output_0"], oracle.gemm_rcr(x, w, b, epilogue="relu"))
    module.close()


def test_dynamic_m_walks_every_gemm_kernel_in_graph_mode(workdir):
    """Two GEMMs with a dynamic M in one model: M = 1..4 take the row-dot kernel, 5..128 the weight-streaming
    tensor-core kernel (N = 8192: clusters of two, N = 1024: clusters of four, every width of the X tile), above that
    the tile kernels. Every size runs eagerly and then twice as a CUDA graph, against the oracle."""
    Model, compile_model, ops, IntVar, Tensor, nn, detect_target = _imports()
    k = 2048
    m_dim = IntVar([1, 512], name="m")
    X = Tensor(shape=[m_dim, k], dtype="float16", name="x", is_input=True)
    R1 = Tensor(shape=[m_dim, 8192], dtype="float16", name="r1", is_input=True)
    W1 = Tensor(shape=[8192, k], dtype="float16", name="w1", is_input=True)
    B1 = Tensor(shape=[8192], dtype="float16", name="b1", is_input=True)
    W2 = Tensor(shape=[1024, 8192], dtype="float16", name="w2", is_input=True)
    B2 = Tensor(shape=[1024], dtype="float16", name="b2", is_input=True)
    H = ops.gemm_rcr_bias_add()(X, W1, B1, R1)
    Y = ops.gemm_rcr_bias_relu()(H, W2, B2)
    Y._attrs["name"], Y._attrs["is_output"] = "y", True
    module = compile_model(Y, detect_target(), workdir, "dyn_m_kernels")
    w1, b1, w2, b2 = _rand((8192, k), 31, 0.02), _rand((8192,), 32), _rand((1024, 8192), 33, 0.02), _rand((1024,), 34)
    fixed = {"w1": w1.cuda(), "b1": b1.cuda(), "w2": w2.cuda(), "b2": b2.cuda()}
    for m in (1, 4, 5, 16, 17, 33, 64, 100, 128, 129, 512):
        x, r1 = _rand((m, k), 40 + m), _rand((m, 8192), 90 + m)
        h = oracle.gemm_rcr(x, w1, b1, r1, epilogue="add").half()
        want = oracle.gemm_rcr(h, w2, b2, epilogue="relu")
        for graph_mode in (False, True, True):
            y = torch.empty((512, 1024), dtype=torch.float16, device="cuda")
            res = module.run_with_tensors(dict(fixed, x=x.cuda(), r1=r1.cuda()), {"y": y}, graph_mode=graph_mode)
            assert tuple(res["y"].shape) == (m, 1024)
            _close(res["y"], want, tol=2e-2)
    module.close()
