"""fuse_mm_elementwise: folds elementwise consumers of a gemm_rcr into its epilogue.

Covers the reference's gemm_rcr patterns (python/aitemplate/compiler/transform/
fuse_mm_elementwise_patterns.py:43-196): gemm_rcr + ADD(1-D bias) -> gemm_rcr_bias;
gemm_rcr_bias + {RELU, GELU, FASTGELU, SIGMOID, TANH, SILU} -> gemm_rcr_bias_<act>;
gemm_rcr_bias + ADD/MUL(tensor of the output's shape) -> gemm_rcr_bias_add / _mul and onwards to
_add_relu, _add_add, _add_add_relu, _mul_add, _mul_tanh, _sigmoid_mul, _sigmoid_mul_tanh.
A GEMM output is only absorbed when the elementwise op is its sole consumer and it is not itself a
graph output.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

from ..base import IntImm, Tensor
from ..ops.common.elementwise import elementwise
from ..ops.common.epilogue import FuncEnum
from ..ops import gemm_universal as G
from .toposort import toposort

_UNARY_NAME = {FuncEnum.RELU: "relu", FuncEnum.GELU: "gelu", FuncEnum.FASTGELU: "fast_gelu",
               FuncEnum.SIGMOID: "sigmoid", FuncEnum.TANH: "tanh", FuncEnum.SILU: "swish"}
_BINARY_NAME = {FuncEnum.ADD: "add", FuncEnum.MUL: "mul"}

# epilogue tuple -> op class (bias present)
_BIAS_CLASSES = {
    ("identity", None, None, "identity"): G.gemm_rcr_bias,
    ("relu", None, None, "identity"): G.gemm_rcr_bias_relu,
    ("gelu", None, None, "identity"): G.gemm_rcr_bias_gelu,
    ("fast_gelu", None, None, "identity"): G.gemm_rcr_bias_fast_gelu,
    ("sigmoid", None, None, "identity"): G.gemm_rcr_bias_sigmoid,
    ("tanh", None, None, "identity"): G.gemm_rcr_bias_tanh,
    ("swish", None, None, "identity"): G.gemm_rcr_bias_swish,
    ("identity", "add", None, "identity"): G.gemm_rcr_bias_add,
    ("identity", "add", None, "relu"): G.gemm_rcr_bias_add_relu,
    ("identity", "add", "add", "identity"): G.gemm_rcr_bias_add_add,
    ("identity", "add", "add", "relu"): G.gemm_rcr_bias_add_add_relu,
    ("identity", "mul", None, "identity"): G.gemm_rcr_bias_mul,
    ("identity", "mul", "add", "identity"): G.gemm_rcr_bias_mul_add,
    ("identity", "mul", None, "tanh"): G.gemm_rcr_bias_mul_tanh,
    ("sigmoid", "mul", None, "identity"): G.gemm_rcr_bias_sigmoid_mul,
    ("sigmoid", "mul", None, "tanh"): G.gemm_rcr_bias_sigmoid_mul_tanh,
}


def _fusable_gemm(op) -> bool:
    return isinstance(op, G.gemm_rcr) and not isinstance(op, (G.gemm_rcr_bias_permute, G.gemm_rcr_permute)) \
        and op._attrs["op"] != "gemm_rcr_fast_gelu"


def _same_shape(a: Tensor, b: Tensor) -> bool:
    return list(a._attrs["shape"]) == list(b._attrs["shape"])


def _next_epilogue(gemm_op, ew: elementwise, out: Tensor) -> Optional[Tuple[type, List[Tensor]]]:
    """Returns (new op class, new input list) if `ew` can be folded into `gemm_op`."""
    func = ew._attrs["func"]
    args = ew._attrs["args"]
    ins = list(gemm_op._attrs["inputs"])
    if not gemm_op._has_bias:
        # gemm_rcr + ADD(out, bias[N]) -> gemm_rcr_bias
        if func == FuncEnum.ADD and len(args) == 2 and gemm_op._epi == ("identity", None, None, "identity"):
            other = args[1] if args[0] is out else args[0]
            n = gemm_op._attrs["inputs"][1]._attrs["shape"][0]
            if not other.is_a_const_num() and other._rank() == 1 and other._attrs["shape"][0] == n \
                    and isinstance(n, IntImm):
                return G.gemm_rcr_bias, ins + [other]
        return None
    u1, b1, b2, u2 = gemm_op._epi
    if func in _UNARY_NAME and len(args) == 1:
        name = _UNARY_NAME[func]
        cand = (name, None, None, "identity") if (b1 is None and u1 == "identity") else (
            (u1, b1, b2, name) if (b1 is not None and u2 == "identity") else None)
        if cand in _BIAS_CLASSES:
            return _BIAS_CLASSES[cand], ins
        return None
    if func in _BINARY_NAME and len(args) == 2:
        other = args[1] if args[0] is out else args[0]
        if other is out or other.is_a_const_num() or not _same_shape(other, out) or u2 != "identity":
            return None
        name = _BINARY_NAME[func]
        cand = (u1, name, None, "identity") if b1 is None else ((u1, b1, name, "identity") if b2 is None else None)
        if cand in _BIAS_CLASSES:
            return _BIAS_CLASSES[cand], ins + [other]
    return None


def fuse_mm_elementwise(sorted_graph: List[Tensor], outputs: Optional[List[Tensor]] = None) -> List[Tensor]:
    """Returns the re-sorted graph. `outputs` (the model's output list, in user order) is updated in
    place when a fused op replaces an output tensor."""
    if outputs is None:
        outputs = [t for t in sorted_graph if t._attrs["is_output"]]
    changed = True
    while changed:
        changed = False
        for t in sorted_graph:
            src = list(t._attrs["src_ops"])
            if len(src) != 1 or not _fusable_gemm(src[0]) or t._attrs["is_output"]:
                continue
            gemm_op = src[0]
            consumers = list(t._attrs["dst_ops"])
            if len(consumers) != 1 or not isinstance(consumers[0], elementwise):
                continue
            ew = consumers[0]
            nxt = _next_epilogue(gemm_op, ew, t)
            if nxt is None:
                continue
            cls, new_inputs = nxt
            old_out = ew._attrs["outputs"][0]
            for x in gemm_op._attrs["inputs"]:
                x._attrs["dst_ops"].discard(gemm_op)
            for x in ew._attrs["inputs"]:
                x._attrs["dst_ops"].discard(ew)
            new_op = cls()
            new_out = new_op(*new_inputs)
            new_out._attrs["name"] = old_out._attrs["name"]
            new_out._attrs["is_output"] = old_out._attrs["is_output"]
            for consumer in list(old_out._attrs["dst_ops"]):
                consumer.replace_input_tensor(old_out, new_out)
                new_out._attrs["dst_ops"].add(consumer)
            if old_out._attrs["is_output"]:
                for i, o in enumerate(outputs):
                    if o is old_out:
                        outputs[i] = new_out
                old_out._attrs["is_output"] = False
            sorted_graph = toposort(outputs)
            changed = True
            break
    return sorted_graph
