"""Strided-output ("memory") fusion into concatenate.

A GEMM or layernorm whose only consumer is a concatenate along the last dim can write its rows straight into
the concatenated buffer: the producer's output TensorAccessor is re-based onto the concat output (element
offset of its column block + the wider row stride), the producer's own tensor becomes an alias of that
buffer, and the concat's input mask for it is cleared so the copy kernel skips it. A concat whose inputs are
all fused launches nothing. This is the "cat pattern" of the reference's pass
(python/aitemplate/compiler/transform/transform_strided_ops.py:94-333, with the accessor arithmetic of
python/aitemplate/compiler/tensor_accessor.py:349-404), restricted to the producers of this path whose kernels
take an output offset and row stride: the gemm and bmm families without a permuted store, and layernorm.
"""
from __future__ import annotations

from typing import List

from ..base import IntImm, Tensor
from .toposort import sorted_ops


def _fusible_producer(op) -> bool:
    from ..ops.gemm_universal.gemm_rcr import gemm
    from ..ops.layernorm import layernorm

    if isinstance(op, gemm):
        return op._attrs.get("layout") is None
    # a layernorm over several trailing dims has rows that span more than the last dim: not a column block
    return isinstance(op, layernorm) and len(op._attrs["normalized_shape"]) == 1


def fuse_strided_cat(sorted_graph: List[Tensor]) -> int:
    """Applies the fusion wherever it is legal; returns the number of concat inputs that were fused."""
    from ..ops.tensor import concatenate

    fused = 0
    for op in sorted_ops(sorted_graph):
        if not isinstance(op, concatenate):
            continue
        out = op._attrs["outputs"][0]
        shape = out._attrs["shape"]
        dim = op._attrs["concat_dim"]
        if dim != len(shape) - 1 or not isinstance(shape[dim], IntImm):
            continue  # rows of the producers must map to rows of the buffer
        inputs = op._attrs["original_inputs"]
        offset = 0
        for i, x in enumerate(inputs):
            xs = x._attrs["shape"]
            if len(xs) != len(shape) or not isinstance(xs[dim], IntImm):
                break  # an empty placeholder or a dynamic width: offsets after it are unknown
            width = xs[dim].value()
            src = list(x._attrs["src_ops"])
            ok = (
                op._attrs["input_masks"][i]
                and len(src) == 1
                and _fusible_producer(src[0])
                and len(src[0]._attrs["outputs"]) == 1
                and set(x._attrs["dst_ops"]) == {op}
                and sum(1 for y in inputs if y is x) == 1
                and not x._attrs["is_output"]
                and x._attrs["is_view_of"] is None
                and src[0]._attrs["output_accessors"][0].stride_dim is None
                and width > 0
            )
            if ok:
                src[0]._attrs["output_accessors"][0].update_base_tensor(out, dim, offset)
                x._attrs["is_view_of"] = out       # same storage; the accessor carries offset and stride
                x._attrs["view_offset_bytes"] = 0
                op._attrs["input_masks"][i] = False
                fused += 1
            offset += width
    return fused


def _strided_reader_slot(op, x):
    """Index of the input accessor through which `op` can read `x` with a row stride, or None: x is operand A of
    a 2-D GEMM, operand B of a gemm_rcr (python/aitemplate/backend/cuda/gemm_universal/gemm_rcr.py:203-232 gives both
    operands an accessor), either operand of a bmm without a permuted store, or the input of a layernorm, and
    appears nowhere else among the op's inputs."""
    from ..ops.gemm_universal.bmm import bmm
    from ..ops.gemm_universal.gemm_rcr import gemm
    from ..ops.layernorm import layernorm

    ins = op._attrs["inputs"]
    if sum(1 for y in ins if y is x) != 1:
        return None
    idx = next(i for i, y in enumerate(ins) if y is x)
    if isinstance(op, bmm):
        ok = idx in (0, 1) and op._attrs.get("layout") is None
    elif isinstance(op, layernorm):
        ok = idx == 0 and len(op._attrs["normalized_shape"]) == 1
    else:
        # operand A of any 2-D GEMM; operand B ([N, K]: a block of K columns) of the gemm_rcr family
        ok = isinstance(op, gemm) and (idx == 0 or (idx == 1 and op._attrs["op"].startswith("gemm_rcr")))
    return idx if ok and op._attrs["input_accessors"][idx].stride_dim is None else None


def fuse_split_strided(sorted_graph: List[Tensor]) -> int:
    """The split side of the reference's strided-op pass (python/aitemplate/compiler/transform/
    transform_strided_ops.py:94-333 together with fuse_split.py): when every consumer of an output of a
    last-dim split is a GEMM (as operand A, or B of a gemm_rcr), a bmm (either operand) or a layernorm, those kernels read their column block of the
    split's input in place: the consumer's input TensorAccessor is re-based onto that input (element
    offset + the wider row stride), the split output becomes an alias of it at the block's byte offset, and
    the split's output mask for it is cleared. A split whose outputs are all fused launches nothing.
    Column blocks must start and end on 16-byte boundaries, the alignment the vector loads and the TMA
    descriptors of the consumers need (the reference checks the same through its alignment attributes).
    Returns the number of split outputs that were fused."""
    from ..dtype import get_dtype_size
    from ..ops.tensor import split

    fused = 0
    for op in sorted_ops(sorted_graph):
        if not isinstance(op, split):
            continue
        x = op._attrs["inputs"][0]
        shape = x._attrs["shape"]
        dim = op._attrs["split_dim"]
        if dim != len(shape) - 1 or not isinstance(shape[dim], IntImm):
            continue
        elem = get_dtype_size(x.dtype())
        offset = 0
        for i, (o, width) in enumerate(zip(op._attrs["outputs"], op._attrs["split_sizes"])):
            readers = list(o._attrs["dst_ops"])
            ok = (
                op._attrs["output_masks"][i]
                and readers
                and not o._attrs["is_output"]
                and o._attrs["is_view_of"] is None
                and width > 0
                and (offset * elem) % 16 == 0
                and (width * elem) % 16 == 0
                and (shape[dim].value() * elem) % 16 == 0
                and all(_strided_reader_slot(r, o) is not None for r in readers)
            )
            if ok:
                for r in readers:
                    r._attrs["input_accessors"][_strided_reader_slot(r, o)].update_base_tensor(x, dim, offset)
                o._attrs["is_view_of"] = x   # same storage: the alias starts at the block's first column
                o._attrs["view_offset_bytes"] = offset * elem
                op._attrs["output_masks"][i] = False
                fused += 1
            offset += width
    return fused


def fuse_gemm_permute0213(sorted_graph: List[Tensor], outputs: List[Tensor]) -> List[Tensor]:
    """gemm -> reshape [B, S, H, d] -> permute (0, 2, 1, 3) becomes one GEMM whose epilogue stores the heads-first
    layout: the GEMM node gets the "Permute4D_0213" layout with shape (S, H) that gemm_rcr_permute carries in the
    reference (python/aitemplate/compiler/ops/gemm_universal/gemm_rcr_permute.py, epilogue functor
    cutlass::layout::Tensor4DPermute0213 of python/aitemplate/backend/cuda/gemm_universal/common_permute.py), and
    the permute's output becomes a reshape view of the GEMM's buffer. This is how the q / k / v projections of an
    attention block reach [B, H, S, d] without a copy kernel. Legal when the GEMM result and the reshape have no
    other reader, nothing on the way is a graph output and every dim is static. Applied only where the permuted
    store is free, i.e. where it can go through the staged TMA store: d a multiple of 64 and S a multiple of 32
    (a 32-row x 64-column box then stays inside one head and one batch entry). With d = 40 (the Stable-Diffusion
    block) the per-vector permuted stores cost what the three copy kernels save (324 against 318 us for the
    block), so those graphs keep their permutes. Returns the re-sorted graph."""
    from ..ops.common.view_ops import reshape
    from ..ops.gemm_universal.bmm import bmm
    from ..ops.gemm_universal.gemm_rcr import gemm, gemm_rrr
    from ..ops.tensor.tensor_ops import _permute_base
    from .toposort import toposort

    changed = True
    while changed:
        changed = False
        for op in sorted_ops(sorted_graph):
            if not isinstance(op, _permute_base) or list(op._attrs["dims"]) != [0, 2, 1, 3]:
                continue
            r = op._attrs["inputs"][0]
            r_src = list(r._attrs["src_ops"])
            if len(r_src) != 1 or not isinstance(r_src[0], reshape) or r._attrs["is_output"]:
                continue
            if set(r._attrs["dst_ops"]) != {op}:
                continue
            x = r_src[0]._attrs["inputs"][0]
            x_src = list(x._attrs["src_ops"])
            if len(x_src) != 1 or x._attrs["is_output"] or set(x._attrs["dst_ops"]) != {r_src[0]}:
                continue
            g = x_src[0]
            if not isinstance(g, gemm) or isinstance(g, (bmm, gemm_rrr)) or g._attrs.get("layout") is not None:
                continue
            if g._attrs["output_accessors"][0].stride_dim is not None:
                continue
            shape = r._attrs["shape"]
            if not all(isinstance(d, IntImm) for d in shape) or not all(isinstance(d, IntImm) for d in x._attrs["shape"]):
                continue
            b, s, h, d = (v.value() for v in shape)
            if x._attrs["shape"][-1].value() != h * d or d % 64 != 0 or s % 32 != 0 or min(b, s, h, d) <= 0:
                continue
            old_out = op._attrs["outputs"][0]
            g._attrs["layout"] = "Permute4D_0213"
            g._attrs["shape"] = (s, h)
            g._attrs["permute_shape"] = f"{s}_{h}"
            x._attrs["dst_ops"].discard(r_src[0])
            new_out = reshape()(x, [b, h, s, d])
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


def fuse_permute_into_attention(sorted_graph: List[Tensor], outputs: List[Tensor]) -> List[Tensor]:
    """permute (0, 2, 1, 3) -> mem_eff_attention becomes the attention alone: the kernel reads an operand stored
    [B, S, H, D] in place through strided tensor maps (row stride H*D, head stride D), so the copy that only
    reorders heads and rows disappears. This is the input-TensorAccessor side of the reference's strided-op fusion
    (python/aitemplate/compiler/transform/transform_strided_ops.py:94-224; the reference's kernel takes q / k / v
    strides, python/aitemplate/backend/cuda/attention/mem_eff_attention.py:160-171) applied to the pattern its
    attention front ends emit (python/aitemplate/frontend/nn/attention.py:360-368: reshape [B, S, H, D] then
    permute). Legal when the permute's output feeds nothing but that attention, is not a graph output, and the
    head size is a multiple of 8 (the strided maps need 16-byte strides). Records `input_layouts` on the op:
    "bshd" for a folded operand, "bhsd" otherwise. Returns the re-sorted graph."""
    from ..ops.attention.mem_eff_attention import mem_eff_attention
    from ..ops.tensor.tensor_ops import _permute_base
    from .toposort import toposort

    changed = False
    for op in sorted_ops(sorted_graph):
        if not isinstance(op, mem_eff_attention) or len(op._attrs["inputs"]) != 3:
            continue  # (with lengths operands the op keeps its contiguous [B, H, S, D] inputs)
        layouts = list(op._attrs.get("input_layouts", ["bhsd"] * 3))
        for i, t in enumerate(list(op._attrs["inputs"][:3])):
            if layouts[i] != "bhsd":
                continue
            src = list(t._attrs["src_ops"])
            if len(src) != 1 or not isinstance(src[0], _permute_base) or list(src[0]._attrs["dims"]) != [0, 2, 1, 3]:
                continue
            if t._attrs["is_output"] or set(t._attrs["dst_ops"]) != {op}:
                continue
            if sum(1 for y in op._attrs["inputs"] if y is t) != 1:
                continue
            head = t._attrs["shape"][3]
            if not isinstance(head, IntImm) or head.value() % 8 != 0 or head.value() > 128:
                continue
            x = src[0]._attrs["inputs"][0]  # stored [B, S, H, D]
            op.replace_input_tensor(t, x)
            x._attrs["dst_ops"].add(op)
            t._attrs["dst_ops"].discard(op)
            op._attrs["input_accessors"][i] = type(op._attrs["input_accessors"][i])(x)
            layouts[i] = "bshd"
            changed = True
        op._attrs["input_layouts"] = layouts
    return toposort(outputs) if changed else sorted_graph
