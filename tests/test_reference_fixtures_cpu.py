"""Replays tests/golden/reference_graph_fixtures.json (recorded from the reference's own Python graph
layer by tests/golden/make_reference_graph_fixtures.py) on aitemplate_b200 and requires the same
output shapes, dtypes, op names and op attributes."""
import json
import os

import pytest

from aitemplate_b200.compiler import ops
from aitemplate_b200.compiler.ops import FuncEnum
from aitemplate_b200.frontend import IntVar, Tensor

FIXTURES = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_graph_fixtures.json")
with open(FIXTURES) as f:
    CASES = json.load(f)


def _describe(d):
    vals = d._attrs["values"]
    return [vals[0], vals[-1]] if len(vals) > 1 and vals[0] != vals[-1] else vals[0]


def _run(case):
    dyn = {}

    def dim(d):
        if isinstance(d, list):
            key = tuple(d)
            if key not in dyn:
                dyn[key] = IntVar(d, name=f"dyn_{len(dyn)}")
            return dyn[key]
        return d

    tensors = [Tensor([dim(d) for d in s], name=f"in_{i}", is_input=True) for i, s in enumerate(case["inputs"])]
    ctor = dict(case["ctor"])
    if "func_enum" in ctor:
        ctor["func_enum"] = FuncEnum[ctor["func_enum"]]
    op = getattr(ops, case["op"])(**ctor)
    call = case["call"]
    name = case["op"]
    if name == "concatenate":
        out = op(tensors, **call)
    elif name == "layernorm":
        out = op(tensors[0], tensors[1], tensors[2], call["normalized_shape"], call["eps"])
    elif name in ("split", "permute", "reshape", "softmax"):
        out = op(tensors[0], **call)
    else:
        out = op(*tensors)
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    node = list(outs[0]._attrs["src_ops"])[0]
    if node._attrs["op"] == "reshape" and name.startswith(("gemm", "bmm")) and name.endswith("permute"):
        node = list(node._attrs["inputs"][0]._attrs["src_ops"])[0]
    return outs, node


@pytest.mark.parametrize("case_name", sorted(CASES.keys()))
def test_matches_reference_graph_layer(case_name):
    case = CASES[case_name]
    outs, node = _run(case)
    assert [[_describe(d) for d in o._attrs["shape"]] for o in outs] == case["output_shapes"]
    assert outs[0]._attrs["dtype"] == case["output_dtype"]
    assert len(node._attrs["inputs"]) == case["num_inputs"]
    for key, want in case["attrs"].items():
        got = node._attrs[key]
        if isinstance(got, tuple):
            got = list(got)
        assert got == want, f"{case_name}: attr {key}: {got!r} != {want!r}"
