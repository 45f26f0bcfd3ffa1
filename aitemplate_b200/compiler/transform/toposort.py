"""toposort / mark_param_tensor / remove_no_ops
(python/aitemplate/compiler/transform/toposort.py, mark_param_tensor.py:52-68, remove_no_ops.py)."""
from __future__ import annotations

from typing import List, Union

from ..base import IntImm, Operator, Tensor


def toposort(nodes: Union[Tensor, List[Tensor]]) -> List[Tensor]:
    """Tensors reachable from the outputs, producers before consumers, deterministic order."""
    if isinstance(nodes, Tensor):
        nodes = [nodes]
    order: List[Tensor] = []
    state = {}
    for root in nodes:
        stack = [(root, False)]
        while stack:
            t, expanded = stack.pop()
            if expanded:
                if state.get(id(t)) != 2:
                    state[id(t)] = 2
                    order.append(t)
                continue
            if id(t) in state:
                continue
            state[id(t)] = 1
            stack.append((t, True))
            for op in reversed(list(t._attrs["src_ops"])):
                for inp in reversed(op._attrs["inputs"]):
                    if id(inp) not in state:
                        stack.append((inp, False))
                # sibling outputs of a multi-output op (split) are part of the graph as well
            view_of = t._attrs["is_view_of"]
            if view_of is not None and id(view_of) not in state:
                stack.append((view_of, False))
    # add sibling outputs of multi-output ops that no output depends on, so the op can still run
    seen = {id(t) for t in order}
    extra = []
    for t in order:
        for op in t._attrs["src_ops"]:
            for o in op._attrs["outputs"]:
                if id(o) not in seen:
                    seen.add(id(o))
                    extra.append(o)
    order.extend(extra)
    return order


def sorted_ops(sorted_graph: List[Tensor]) -> List[Operator]:
    """Operators in execution order."""
    ops: List[Operator] = []
    seen = set()
    for t in sorted_graph:
        for op in t._attrs["src_ops"]:
            if id(op) not in seen:
                seen.add(id(op))
                ops.append(op)
    return ops


def mark_param_tensor(sorted_graph: List[Tensor]) -> None:
    """Tensors without a producer that are not inputs are constants (is_param)."""
    for t in sorted_graph:
        if t.is_a_const_num():
            continue
        if not t._attrs["src_ops"] and not t._attrs["is_input"]:
            t._attrs["is_param"] = True


def remove_no_ops(sorted_graph: List[Tensor]) -> List[Tensor]:
    """Drops ops that produce nothing observable: a split with a single full-size output becomes the
    input itself for its consumers; zero-element concatenate inputs are dropped from the op."""
    from ..ops.tensor import concatenate

    for t in sorted_graph:
        for op in list(t._attrs["dst_ops"]):
            if isinstance(op, concatenate) and len(op._attrs["inputs"]) > 1:
                keep = []
                for i, x in enumerate(op._attrs["inputs"]):
                    dim = op._attrs["concat_dim"]
                    shape = x._attrs["shape"]
                    empty = len(shape) == 1 and shape[0] == IntImm(0) or (
                        len(shape) > dim and shape[dim] == IntImm(0))
                    keep.append(not empty)
                if not all(keep) and any(keep):
                    for x, k in zip(op._attrs["inputs"], keep):
                        if not k:
                            x._attrs["dst_ops"].discard(op)
                    op._attrs["inputs"] = [x for x, k in zip(op._attrs["inputs"], keep) if k]
                    op._attrs["original_inputs"] = list(op._attrs["inputs"])
                    op._attrs["input_masks"] = [True] * len(op._attrs["inputs"])
    return sorted_graph


def split_to_views(sorted_graph: List[Tensor]) -> None:
    """A split along the outermost non-unit dim yields contiguous slices: its outputs become views
    of the input at a byte offset and nothing is copied (what the reference's fuse_split pass achieves
    for its consumers, python/aitemplate/compiler/transform/fuse_split.py). Outputs that are graph
    outputs keep the copying kernel."""
    from ..dtype import get_dtype_size
    from ..ops.tensor import split

    for op in sorted_ops(sorted_graph):
        if not isinstance(op, split):
            continue
        x = op._attrs["inputs"][0]
        dim = op._attrs["split_dim"]
        shape = x._attrs["shape"]
        if any(not (isinstance(d, IntImm) and d.value() == 1) for d in shape[:dim]):
            continue
        if any(not isinstance(d, IntImm) for d in shape[dim + 1:]):
            continue
        if any(o._attrs["is_output"] for o in op._attrs["outputs"]):
            continue
        inner = get_dtype_size(x.dtype())
        for d in shape[dim + 1:]:
            inner *= d.value()
        off = 0
        for i, (o, size) in enumerate(zip(op._attrs["outputs"], op._attrs["split_sizes"])):
            o._attrs["is_view_of"] = x
            o._attrs["view_offset_bytes"] = off
            op._attrs["output_masks"][i] = False
            off += size * inner
