"""`import aitemplate` answers with this package: the reference's import statements work unchanged.

The contract is python/aitemplate/compiler/__init__.py and compiler/ops/__init__.py:20-37 of the reference
(`from aitemplate.compiler import compile_model, ops, Model`, flat op export) and the idiom of its tests
(tests/unittest/ops/test_gemm_rcr_bias_fast_gelu.py:72-77). Where a reference checkout is present, the
reference's own examples/03_bert/modeling/bert.py is loaded AS IS (its only imports are `aitemplate.*`) and its
BertEncoder is built; otherwise that part is skipped and an encoder layer written with the same imports is
built instead.
"""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_BERT = "/root/reference/examples/03_bert/modeling/bert.py"


def test_reference_import_statements_resolve_to_this_package():
    import aitemplate
    import aitemplate_b200
    from aitemplate.compiler import compile_model, Model, ops  # noqa: F401
    from aitemplate.compiler.base import IntImm, IntVar, IntVarTensor  # noqa: F401
    from aitemplate.compiler.ops.common.epilogue import FuncEnum
    from aitemplate.frontend import IntImm as I2, IntVar as V2, nn, Tensor  # noqa: F401
    from aitemplate.testing import benchmark_pt, detect_target  # noqa: F401
    from aitemplate.testing.test_utils import (  # noqa: F401
        env_variables,
        filter_test_cases_by_params,
        filter_test_cases_by_test_env,
        get_random_torch_tensor,
        get_torch_empty_tensor,
        TestEnv,
    )
    from aitemplate.utils import shape_utils
    from aitemplate.utils.torch_utils import string_to_torch_dtype, torch_dtype_to_string

    assert os.path.dirname(aitemplate.__file__) == os.path.join(ROOT, "aitemplate")
    assert aitemplate.compiler is aitemplate_b200.compiler and ops is aitemplate_b200.compiler.ops
    assert sys.modules["aitemplate.compiler.ops"] is sys.modules["aitemplate_b200.compiler.ops"]
    assert FuncEnum.ADD.value == 1 and I2 is IntImm
    assert torch_dtype_to_string(string_to_torch_dtype("float16")) == "float16"
    assert shape_utils.gen_int_var([3, 1, 3])._attrs["values"] == [1, 3]
    for name in ("gemm_rcr", "gemm_rcr_bias", "gemm_rcr_bias_fast_gelu", "gemm_rcr_bias_add", "gemm_rcr_bias_permute",
                 "bmm_rcr", "mem_eff_attention", "flash_attention", "layernorm", "softmax", "elementwise", "concatenate",
                 "split", "permute", "reshape", "flatten", "squeeze", "unsqueeze"):
        assert hasattr(ops, name), name
    with pytest.raises(ModuleNotFoundError):
        import aitemplate.backend.rocm  # noqa: F401
    assert detect_target().name() == "cuda"
    cases = filter_test_cases_by_params({TestEnv.CUDA_LESS_THAN_SM80: [("a",)], TestEnv.CUDA_SM80: [("b",)],
                                         TestEnv.ROCM: [("c",)]})
    assert cases == [("a",), ("b",)]


def test_reference_test_idiom_builds_a_graph():
    from aitemplate.compiler import ops
    from aitemplate.frontend import IntVar, Tensor

    m = IntVar([1, 128], name="M")
    X = Tensor(shape=[m, 1024], dtype="float16", name="input_0", is_input=True)
    W = Tensor(shape=[64, 1024], dtype="float16", name="input_1", is_input=True)
    B = Tensor(shape=[64], dtype="float16", name="input_2", is_input=True)
    Y = ops.gemm_rcr_bias_fast_gelu()(X, W, B)
    Y._attrs["name"] = "output_0"
    Y._attrs["is_output"] = True
    assert [d._attrs["values"] for d in Y._attrs["shape"]] == [[1, 128], [64]]


def _layer_kernels(hidden_states_out):
    from test_graph_cpu import _lower

    _, plan, _, _ = _lower([hidden_states_out])
    return [l.split()[1] for l in plan.splitlines() if l.startswith("op ") and l.split()[1] != "view"]


@pytest.mark.skipif(not os.path.exists(REFERENCE_BERT), reason="needs the reference checkout")
def test_reference_bert_example_builds_unmodified():
    """examples/03_bert/modeling/bert.py:112-200 (BertLayer / BertEncoder), loaded from the reference as is."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("reference_bert_model", REFERENCE_BERT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    from aitemplate.frontend import Tensor

    batch, seq, hidden = 4, 384, 768
    enc = mod.BertEncoder(num_hidden_layers=2, hidden_size=hidden, batch_size=batch, seq_len=seq, num_attention_heads=12,
                          intermediate_size=3072, hidden_act="fast_gelu", layer_norm_eps=1e-12,
                          attention_probs_dropout_prob=0.0, hidden_dropout_prob=0.0)
    enc.name_parameter_tensor()
    x = Tensor([batch, seq, hidden], name="hidden_states", is_input=True)
    (y,) = enc(x)
    y._attrs["name"], y._attrs["is_output"] = "output_0", True
    assert [d.value() for d in y._attrs["shape"]] == [batch, seq, hidden]
    layer = ["gemm_rcr", "flash_attention", "gemm_rcr", "layernorm", "gemm_rcr", "gemm_rcr", "layernorm"]
    assert _layer_kernels(y) == layer * 2
    names = {p.tensor()._attrs["name"] for p in enc.parameters()}
    assert "layer_0_attention_self_cu_length" in names and "layer_1_output_dense_weight" in names


def test_encoder_layer_written_against_the_alias_takes_the_flash_path():
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from aitemplate.compiler import ops
    from aitemplate.frontend import nn, Tensor

    batch, seq, hidden, heads = 2, 128, 256, 4
    attn = nn.MultiheadAttention(dim=hidden, batch_size=batch, seq_len=seq, num_heads=heads, qkv_bias=True,
                                 has_residual=True)
    assert attn.use_flash and isinstance(attn.op, ops.flash_attention)
    ln = nn.LayerNorm(hidden, eps=1e-12)
    x = Tensor([batch, seq, hidden], name="hidden_states", is_input=True)
    y = ln(attn(x, x))
    y._attrs["name"], y._attrs["is_output"] = "output_0", True
    assert _layer_kernels(y) == ["gemm_rcr", "flash_attention", "gemm_rcr", "layernorm"]
    fa = attn.op
    assert fa._attrs["head_size"] == 64 and fa._attrs["seq_len"] == 128
    assert fa._get_op_attributes() == {"batch_size": batch, "dropout": 0.0, "max_seq_len": seq, "causal": False}
    out = fa._attrs["outputs"][0]
    assert [d.value() for d in out._attrs["shape"]] == [batch * seq, heads, 64]
    mem = nn.MultiheadAttention(dim=hidden, batch_size=batch, seq_len=seq, num_heads=heads, use_mem_eff=True)
    assert isinstance(mem.op, ops.mem_eff_attention) and mem.qkv._op_name == "gemm_rcr_bias_permute"
