"""Generates tests/golden/reference_graph_fixtures.json by importing the REFERENCE's Python graph
layer (python/aitemplate under the reference checkout) and recording, for a set of op calls, the
output shapes and the op attributes that the hot path depends on.

Run in a container that has the reference checkout:
    AIT_BUILD_DOCS=1 PYTHONPATH=<reference>/python python tests/golden/make_reference_graph_fixtures.py
AIT_BUILD_DOCS makes the reference's detect_target() return a CUDA sm80 target without a GPU
(python/aitemplate/testing/detect_target.py:116-118). The fixtures are consumed by
tests/test_reference_fixtures_cpu.py, which replays the same calls on aitemplate_b200.
"""
import json
import os
import sys

CASES = [
    # (case name, op name, constructor kwargs, input shapes (lists; [lo, hi] pairs are dynamic dims), call kwargs)
    ("gemm_rcr_2d", "gemm_rcr", {}, [[256, 768], [3072, 768]], {}),
    ("gemm_rcr_3d_dynamic", "gemm_rcr", {}, [[[1, 64], 384, 768], [2304, 768]], {}),
    ("gemm_rcr_bias", "gemm_rcr_bias", {}, [[4096, 1024], [81, 1024], [81]], {}),
    ("gemm_rcr_bias_relu", "gemm_rcr_bias_relu", {}, [[128, 64], [1024, 64], [1024]], {}),
    ("gemm_rcr_bias_gelu", "gemm_rcr_bias_gelu", {}, [[128, 1024], [64, 1024], [64]], {}),
    ("gemm_rcr_bias_fast_gelu", "gemm_rcr_bias_fast_gelu", {}, [[[1, 127], 1024], [64, 1024], [64]], {}),
    ("gemm_rcr_bias_sigmoid", "gemm_rcr_bias_sigmoid", {}, [[16, 8], [8, 8], [8]], {}),
    ("gemm_rcr_bias_tanh", "gemm_rcr_bias_tanh", {}, [[16, 8], [8, 8], [8]], {}),
    ("gemm_rcr_bias_swish", "gemm_rcr_bias_swish", {}, [[16, 8], [8, 8], [8]], {}),
    ("gemm_rcr_bias_hardswish", "gemm_rcr_bias_hardswish", {}, [[16, 8], [8, 8], [8]], {}),
    ("gemm_rcr_bias_add", "gemm_rcr_bias_add", {}, [[8, 8], [8, 8], [8], [8, 8]], {}),
    ("gemm_rcr_bias_add_relu", "gemm_rcr_bias_add_relu", {}, [[[2, 32], 256], [128, 256], [128], [[2, 32], 128]], {}),
    ("gemm_rcr_bias_mul", "gemm_rcr_bias_mul", {}, [[8192, 320], [1280, 320], [1280], [8192, 1280]], {}),
    ("gemm_rcr_bias_add_add", "gemm_rcr_bias_add_add", {}, [[21, 1024], [512, 1024], [512], [21, 512], [21, 512]], {}),
    ("gemm_rcr_bias_add_add_relu", "gemm_rcr_bias_add_add_relu", {}, [[8, 8], [8, 8], [8], [8, 8], [8, 8]], {}),
    ("gemm_rcr_bias_mul_add", "gemm_rcr_bias_mul_add", {}, [[8, 8], [8, 8], [8], [8, 8], [8, 8]], {}),
    ("gemm_rcr_bias_mul_tanh", "gemm_rcr_bias_mul_tanh", {}, [[8, 8], [8, 8], [8], [8, 8]], {}),
    ("gemm_rcr_bias_sigmoid_mul", "gemm_rcr_bias_sigmoid_mul", {}, [[8, 8], [8, 8], [8], [8, 8]], {}),
    ("gemm_rcr_bias_sigmoid_mul_tanh", "gemm_rcr_bias_sigmoid_mul_tanh", {}, [[8, 8], [8, 8], [8], [8, 8]], {}),
    ("gemm_rcr_bias_permute_bert", "gemm_rcr_bias_permute", {"shape": [384, 3, 12]}, [[24576, 768], [2304, 768], [2304]], {}),
    ("gemm_rcr_bias_permute_small", "gemm_rcr_bias_permute", {"shape": [8, 3, 4]}, [[128, 80], [240, 80], [240]], {}),
    ("gemm_rcr_permute_0213", "gemm_rcr_permute", {"shape": [96, 8], "layout": "0213"}, [[192, 320], [320, 320]], {}),
    ("bmm_rcr", "bmm_rcr", {}, [[1024, 512, 64], [1024, 512, 64]], {}),
    ("bmm_rcr_dynamic_batch", "bmm_rcr", {}, [[[1, 977], 100, 256], [[1, 977], 512, 256]], {}),
    ("bmm_rcr_broadcast_b", "bmm_rcr", {}, [[5, 32, 256], [1, 512, 256]], {}),
    ("bmm_rcr_2d_b", "bmm_rcr", {}, [[5, 32, 256], [512, 256]], {}),
    ("gemm_rrr", "gemm_rrr", {}, [[[1, 1024], 256], [256, 384]], {}),
    ("gemm_rrr_3d_a", "gemm_rrr", {}, [[4, 17, 64], [64, 72]], {}),
    ("gemm_rrr_bias", "gemm_rrr_bias", {}, [[1000, 128], [128, 264], [264]], {}),
    ("bmm_rrr", "bmm_rrr", {}, [[16, 384, 384], [16, 384, 64]], {}),
    ("bmm_rrr_dynamic_batch", "bmm_rrr", {}, [[[1, 64], 48, 40], [[1, 64], 40, 24]], {}),
    ("bmm_rrr_broadcast_b", "bmm_rrr", {}, [[5, 32, 256], [1, 256, 72]], {}),
    ("bmm_rcr_permute", "bmm_rcr_permute", {"shape": [12]}, [[24, 80, 88], [24, 64, 88]], {}),
    ("bmm_rrr_permute", "bmm_rrr_permute", {"shape": [10]}, [[100, 88, 64], [100, 64, 88]], {}),
    ("mem_eff_attention", "mem_eff_attention", {"causal": False}, [[64, 12, 384, 64]] * 3, {}),
    ("mem_eff_attention_cross", "mem_eff_attention", {"causal": False},
     [[2, 8, 4096, 40], [2, 8, 77, 40], [2, 8, 77, 40]], {}),
    ("mem_eff_attention_dynamic", "mem_eff_attention", {"causal": True}, [[[1, 16], 4, 8, 20]] * 3, {}),
    ("layernorm", "layernorm", {}, [[[1, 1024], 1496], [1496], [1496]], {"normalized_shape": [1496], "eps": 1e-5}),
    ("layernorm_2d_norm", "layernorm", {}, [[7, 5, 16, 24], [16, 24], [16, 24]], {"normalized_shape": [16, 24], "eps": 0.1}),
    ("softmax_last", "softmax", {}, [[512, 1024, 1024]], {"dim": -1}),
    ("softmax_mid", "softmax", {}, [[[1, 4], 33, 5]], {"dim": 1}),
    ("concatenate_dim1", "concatenate", {}, [[8192, 1024]] * 4, {"dim": 1}),
    ("concatenate_dynamic", "concatenate", {}, [[[1, 8], 3, 4], [[1, 8], 5, 4]], {"dim": 1}),
    ("concatenate_dynamic_cat_dim", "concatenate", {}, [[[2, 6], 4], [[3, 9], 4]], {"dim": 0}),
    ("split_sections", "split", {}, [[8192, 4096]], {"split_size_or_sections": [1024, 1024, 1024, 1024], "dim": 1}),
    ("split_size_ragged", "split", {}, [[3, 10, 2]], {"split_size_or_sections": 4, "dim": 1}),
    ("split_dim0", "split", {}, [[3, 64, 12, 384, 64]], {"split_size_or_sections": 1, "dim": 0}),
    ("permute_0213", "permute", {}, [[2, 4096, 8, 40]], {"dims": [0, 2, 1, 3]}),
    ("permute_5d", "permute", {}, [[[1, 4], 3, 4, 5, 6]], {"dims": [4, 0, 3, 1, 2]}),
    ("permute021", "permute021", {}, [[3, 5, 7]], {}),
    ("permute102", "permute102", {}, [[3, 5, 7]], {}),
    ("permute210", "permute210", {}, [[3, 5, 7]], {}),
    ("permute0213", "permute0213", {}, [[2, 3, 5, 7]], {}),
    ("reshape_minus1", "reshape", {}, [[[1, 64], 384, 768]], {"shape": [-1, 768]}),
    ("reshape_static", "reshape", {}, [[24576, 768]], {"shape": [64, 384, 12, 64]}),
    ("flatten", "flatten", {"start_dim": 1, "end_dim": -1}, [[[1, 8], 3, 4, 5]], {}),
    ("flatten_all", "flatten", {}, [[2, 3, 4]], {}),
    ("squeeze", "squeeze", {"dim": 1}, [[4, 1, 6]], {}),
    ("squeeze_none", "squeeze", {"dim": None}, [[1, 4, 1, 6]], {}),
    ("unsqueeze", "unsqueeze", {"dim": -1}, [[4, 6]], {}),
    ("elementwise_add_broadcast", "elementwise", {"func_enum": "ADD"}, [[[1, 8], 4096, 320], [320]], {}),
    ("elementwise_mul_broadcast", "elementwise", {"func_enum": "MUL"}, [[4, 1, 8], [1, 5, 8]], {}),
    ("elementwise_gelu", "elementwise", {"func_enum": "GELU"}, [[16, 64]], {}),
]

ATTR_KEYS = ["op", "epilogue", "num_sources", "alpha", "split_k", "shape", "layout", "causal", "head_size", "eps",
             "dim", "concat_dim", "split_dim", "split_sizes", "dims", "input_masks", "output_masks"]


def describe_dim(d):
    vals = d._attrs["values"]
    return [vals[0], vals[-1]] if len(vals) > 1 and vals[0] != vals[-1] else vals[0]


def run_case(ops, Tensor, IntVar, FuncEnum, case):
    name, op_name, ctor, in_shapes, call_kwargs = case
    dyn = {}

    def dim(d, i, j):
        if isinstance(d, list):
            key = tuple(d)
            if key not in dyn:
                dyn[key] = IntVar(d, name=f"dyn_{len(dyn)}")
            return dyn[key]
        return d

    tensors = [Tensor([dim(d, i, j) for j, d in enumerate(s)], name=f"in_{i}", is_input=True)
               for i, s in enumerate(in_shapes)]
    ctor = dict(ctor)
    if "func_enum" in ctor:
        ctor["func_enum"] = FuncEnum[ctor["func_enum"]]
    op = getattr(ops, op_name)(**ctor)
    if op_name == "concatenate":
        out = op(tensors, **call_kwargs)
    elif op_name == "layernorm":
        out = op(tensors[0], tensors[1], tensors[2], call_kwargs["normalized_shape"], call_kwargs["eps"])
    elif op_name in ("split", "permute", "reshape", "softmax"):
        out = op(tensors[0], **call_kwargs)
    else:
        out = op(*tensors)
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    src = list(outs[0]._attrs["src_ops"])[0]
    # the *_permute GEMMs return a reshape of the GEMM output: record the GEMM's attrs
    node = src
    if src._attrs["op"] == "reshape" and op_name.endswith("permute") and op_name.startswith(("gemm", "bmm")):
        node = list(src._attrs["inputs"][0]._attrs["src_ops"])[0]
    attrs = {}
    for k in ATTR_KEYS:
        if k in node._attrs:
            v = node._attrs[k]
            if k == "shape" and node._attrs["op"] in ("reshape",):
                continue
            if k in ("shape",):
                v = list(v)
            if isinstance(v, tuple):
                v = list(v)
            attrs[k] = v
    return {
        "op": op_name, "ctor": case[2], "inputs": in_shapes, "call": call_kwargs,
        "output_shapes": [[describe_dim(d) for d in o._attrs["shape"]] for o in outs],
        "output_dtype": outs[0]._attrs["dtype"], "attrs": attrs,
        "num_inputs": len(node._attrs["inputs"]),
    }


def main():
    from aitemplate.compiler import ops
    from aitemplate.compiler.ops.common.epilogue import FuncEnum
    from aitemplate.frontend import IntVar, Tensor

    import aitemplate

    assert "reference" in os.path.abspath(aitemplate.__file__), "this script must import the reference package"
    out = {}
    for case in CASES:
        out[case[0]] = run_case(ops, Tensor, IntVar, FuncEnum, case)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_graph_fixtures.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(f"wrote {len(out)} cases to {path}")


if __name__ == "__main__":
    main()
