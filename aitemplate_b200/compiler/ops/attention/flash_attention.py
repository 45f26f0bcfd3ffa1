"""flash_attention graph node: packed-QKV, variable-length multi-head attention
(python/aitemplate/compiler/ops/attention/flash_attention.py:49-196).

    y = flash_attention(batch_size, dropout, max_seq_len, causal)(qkv, cu_seqlens)

qkv is [total, 3, num_heads, head_size] (the rows of all sequences back to back), cu_seqlens the
int32 [batch_size + 1] cumulative row offsets; sequence b owns rows cu_seqlens[b] .. cu_seqlens[b+1]
and attends only to itself. The output is [total, num_heads, head_size]. The softmax scale is
1 / sqrt(head_size) (python/aitemplate/backend/cuda/attention/flash_attention.py:267-300).

The reference lowers this to its own FMHA kernels; here it is the same tensor-core attention kernel
as mem_eff_attention, reading q, k and v in place from the packed tensor through strided tensor
maps, so no split or permute copy is made."""
from __future__ import annotations

import math
from typing import Any, Dict, List

from ...base import IntImm, IntVar, Operator, Tensor
from ...tensor_accessor import TensorAccessor


class flash_attention(Operator):
    def __init__(self, batch_size, dropout, max_seq_len, causal) -> None:
        super().__init__()
        assert dropout == 0
        self._attrs["op"] = "flash_attention"
        self._attrs["has_profiler"] = False
        self._attrs["batch_size"] = batch_size
        self._attrs["dropout"] = dropout
        self._attrs["max_seq_len"] = max_seq_len
        self._attrs["seq_len"] = 512
        self._attrs["head_size"] = -1
        self._attrs["causal"] = causal
        self._attrs["workspace"] = 0

    def _get_op_attributes(self):
        return {k: self._attrs[k] for k in ("batch_size", "dropout", "max_seq_len", "causal")}

    def _infer_shapes(self, x: Tensor, cu_seqlens: Tensor) -> List[IntVar]:
        xs = x._attrs["shape"]
        return [xs[0], xs[2], xs[3]]  # NO = total, HO = num_heads, WO = head_size (flash_attention.py:30-38)

    def __call__(self, x: Tensor, cu_seqlens: Tensor) -> Tensor:
        if x._rank() != 4:
            raise RuntimeError("flash_attention: qkv must be [total, 3, num_heads, head_size]")
        three, heads, head = x._attrs["shape"][1:]
        if not all(isinstance(d, IntImm) for d in (three, heads, head)) or three.value() != 3:
            raise RuntimeError("flash_attention: qkv must be [total, 3, num_heads, head_size] with static trailing dims")
        if cu_seqlens._rank() != 1 or cu_seqlens.dtype() not in ("int32", "int"):
            raise RuntimeError("flash_attention: cu_seqlens must be an int32 vector of batch_size + 1 entries")
        n = cu_seqlens._attrs["shape"][0]
        if isinstance(n, IntImm) and n.value() != self._attrs["batch_size"] + 1:
            raise RuntimeError(f"flash_attention: cu_seqlens has {n.value()} entries, expected batch_size + 1 = "
                               f"{self._attrs['batch_size'] + 1}")
        head_size = head.value()
        assert head_size in [8, 16, 32, 64, 128]  # the head sizes the reference op accepts (flash_attention.py:153)
        self._attrs["head_size"] = head_size
        max_seq_len = self._attrs["max_seq_len"]
        # the reference rounds the sequence length up to its kernel's tile (flash_attention.py:156-163); kept as an
        # attribute only, this kernel masks by the true lengths
        base_n = 256
        self._attrs["seq_len"] = 128 if max_seq_len <= 128 else 256 if max_seq_len <= 256 else \
            ((max_seq_len + base_n - 1) // base_n) * base_n
        self._attrs["inputs"] = [x, cu_seqlens]
        self._attrs["input_accessors"] = [TensorAccessor(t) for t in self._attrs["inputs"]]
        self._set_depth()
        out = Tensor(self._infer_shapes(x, cu_seqlens), src_ops={self}, dtype=x.dtype())
        self._attrs["outputs"] = [out]
        self._attrs["output_accessors"] = [TensorAccessor(out)]
        return out

    def _lower(self) -> Dict[str, Any]:
        d = self._attrs["head_size"]
        return {"kernel": "flash_attention", "operands": list(self._attrs["inputs"]),
                "ints": [1 if self._attrs["causal"] else 0, int(self._attrs["batch_size"]),
                         int(self._attrs["max_seq_len"])],
                "floats": [1.0 / math.sqrt(d) if d else 1.0]}
