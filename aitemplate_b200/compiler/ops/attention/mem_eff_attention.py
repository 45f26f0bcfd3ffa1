"""mem_eff_attention graph node: softmax(Q K^T / sqrt(d)) V with q, k, v [B, H, S, D] and output
[B, Sq, H, Dv] (python/aitemplate/compiler/ops/attention/mem_eff_attention.py:50-263). The softmax
scale is always 1/sqrt(head_size), as in the reference kernel (kernel_forward.h:655). With
variable_seq_length_kv / variable_seq_length_q the op takes int32 tensors of batch_size lengths: batch b attends to
its first lengths_kv[b] keys, and only its first lengths_q[b] query rows are computed and written
(kernel_forward.h:183-197; tests/unittest/ops/test_attention.py:504-530)."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

from ...base import IntImm, IntVar, Operator, Tensor
from ...tensor_accessor import TensorAccessor


class mem_eff_attention(Operator):
    def __init__(self, causal, dropout=0, variable_seq_length_kv=False, variable_seq_length_q=False,
                 use_grouped_fmha=False) -> None:
        super().__init__()
        assert dropout == 0
        # use_grouped_fmha selects another kernel template with the same signature and results in the reference
        # (backend/cuda/attention/mem_eff_attention.py:694-697); here one kernel already schedules (batch, head,
        # query tile) items with per-item sizes, so the flag is kept as an attribute and changes nothing
        self._attrs["op"] = "mem_eff_attention"
        self._attrs["has_profiler"] = False
        self._attrs["dropout"] = dropout
        self._attrs["causal"] = causal
        self._attrs["variable_seq_length_kv"] = variable_seq_length_kv
        self._attrs["variable_seq_length_q"] = variable_seq_length_q
        self._attrs["head_size"] = -1
        self._attrs["workspace"] = 0
        self._attrs["use_grouped_fmha"] = use_grouped_fmha

    def _get_op_attributes(self):
        return {"causal": self._attrs["causal"], "dropout": self._attrs["dropout"],
                "variable_seq_length_kv": self._attrs["variable_seq_length_kv"],
                "variable_seq_length_q": self._attrs["variable_seq_length_q"],
                "use_grouped_fmha": self._attrs["use_grouped_fmha"]}

    def _infer_shapes(self, q: Tensor, v: Tensor) -> List[IntVar]:
        qs = q._attrs["shape"]
        return [qs[0], qs[2], qs[1], v._attrs["shape"][-1]]

    def __call__(self, q: Tensor, k: Tensor, v: Tensor, lengths_kv: Optional[Tensor] = None,
                 lengths_q: Optional[Tensor] = None) -> Tensor:
        for flag, t, name in ((self._attrs["variable_seq_length_kv"], lengths_kv, "lengths_kv"),
                              (self._attrs["variable_seq_length_q"], lengths_q, "lengths_q")):
            if flag and t is None:
                raise RuntimeError(f"mem_eff_attention: {name} is required by the variable_seq_length flag")
            if flag and t.dtype() not in ("int", "int32"):
                raise RuntimeError(f"mem_eff_attention: {name} must be an int32 tensor")
        for name, t in (("q", q), ("k", k), ("v", v)):
            if t._rank() != 4:
                raise RuntimeError(f"mem_eff_attention: {name} must be [batch, heads, seq, head_size]")
        head = q._attrs["shape"][3]
        if not isinstance(head, IntImm):
            raise RuntimeError("mem_eff_attention: head size must be static")
        if k._attrs["shape"][3] != head:
            raise RuntimeError("mem_eff_attention: q and k head sizes differ")
        if k._attrs["shape"][2] != v._attrs["shape"][2]:
            raise RuntimeError("mem_eff_attention: k and v sequence lengths differ")
        self._attrs["head_size"] = head.value()
        self._attrs["inputs"] = [q, k, v]
        # as in the reference, a lengths tensor is only an input when its flag is set (a stray argument is ignored)
        if self._attrs["variable_seq_length_kv"]:
            self._attrs["inputs"].append(lengths_kv)
        if self._attrs["variable_seq_length_q"]:
            self._attrs["inputs"].append(lengths_q)
        self._attrs["input_accessors"] = [TensorAccessor(t) for t in self._attrs["inputs"]]
        self._set_depth()
        out = Tensor(self._infer_shapes(q, v), src_ops={self}, dtype=q.dtype())
        self._attrs["outputs"] = [out]
        self._attrs["output_accessors"] = [TensorAccessor(out)]
        return out

    def _lower(self) -> Dict[str, Any]:
        d = self._attrs["head_size"]
        # input_layouts: set by fuse_permute_into_attention; "bshd" = the operand is stored [B, S, H, D] and read in place
        layouts = self._attrs.get("input_layouts", ["bhsd"] * 3)
        return {"kernel": "mem_eff_attention", "operands": list(self._attrs["inputs"]),
                # causal, three storage flags, then whether a lengths_kv / a lengths_q operand follows q, k, v
                "ints": [1 if self._attrs["causal"] else 0] + [1 if l == "bshd" else 0 for l in layouts[:3]]
                + [1 if self._attrs["variable_seq_length_kv"] else 0, 1 if self._attrs["variable_seq_length_q"] else 0],
                "floats": [1.0 / math.sqrt(d) if d else 1.0]}
