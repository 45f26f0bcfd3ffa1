"""memory_planning: packs intermediate tensors into one activation blob.

Greedy-by-size interval colouring over tensor lifetimes, as the reference does
(python/aitemplate/compiler/transform/memory_planning.py:53-290): tensors are sized at the upper
bound of every dim, views share their base's storage, and two tensors may overlap in the blob only
when their lifetimes (first write .. last read, in op order) are disjoint. Constants go to a
separate slab. Offsets are 256-byte aligned so every tensor is a legal TMA base address."""
from __future__ import annotations

from typing import Dict, List, Tuple

from ..base import Tensor
from .toposort import sorted_ops

ALIGN = 256


def storage_root(t: Tensor) -> Tensor:
    while t._attrs["is_view_of"] is not None:
        t = t._attrs["is_view_of"]
    return t


def _aligned(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def memory_planning(sorted_graph: List[Tensor]) -> Tuple[int, int]:
    """Sets `_attrs["offset"]` on constants (into the constants slab) and on intermediate storage
    tensors (into the blob). Returns (blob_bytes, constants_bytes)."""
    ops = sorted_ops(sorted_graph)
    op_index = {id(op): i for i, op in enumerate(ops)}
    first: Dict[int, int] = {}
    last: Dict[int, int] = {}
    roots: Dict[int, Tensor] = {}
    for t in sorted_graph:
        if t.is_a_const_num():
            continue
        r = storage_root(t)
        roots[id(r)] = r
        for op in t._attrs["src_ops"]:
            i = op_index[id(op)]
            first[id(r)] = min(first.get(id(r), i), i)
            last[id(r)] = max(last.get(id(r), i), i)
        for op in t._attrs["dst_ops"]:
            if id(op) in op_index:
                i = op_index[id(op)]
                last[id(r)] = max(last.get(id(r), i), i)
    const_off = 0
    for t in sorted_graph:
        if t._attrs["is_param"] and t._attrs["is_view_of"] is None:
            t._attrs["offset"] = const_off
            const_off += _aligned(t.size_bytes())
    # intermediates: storage roots that are neither inputs, constants, nor (aliases of) outputs
    cands = []
    for r in roots.values():
        if r._attrs["is_input"] or r._attrs["is_param"] or r._attrs.get("output_slot") is not None:
            continue
        size = _aligned(r.size_bytes())
        cands.append((size, first.get(id(r), 0), last.get(id(r), len(ops)), r))
    cands.sort(key=lambda c: (-c[0], c[1]))
    placed: List[Tuple[int, int, int, int]] = []  # (offset, size, first, last)
    blob = 0
    for size, f, l, r in cands:
        conflicts = sorted((o, s) for (o, s, pf, pl) in placed if not (pl < f or l < pf))
        off = 0
        for o, s in conflicts:
            if off + size <= o:
                break
            off = max(off, o + s)
        r._attrs["offset"] = off
        placed.append((off, size, f, l))
        blob = max(blob, off + size)
    return blob, const_off
