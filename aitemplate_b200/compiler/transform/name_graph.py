"""name_graph: gives every op, tensor and dynamic dim a unique C-identifier-safe name
(python/aitemplate/compiler/transform/name_graph.py:62-150). Unnamed ops become `<op>_<n>`, their
unnamed outputs `<func>_<k>`, unnamed source tensors `tensor_<n>`, unnamed dims `<tensor>_dim_<i>`."""
from __future__ import annotations

import re
from typing import Dict, List

from ..base import IntImm, Tensor
from .toposort import sorted_ops

_counters = {"func": 0, "tensor": 0}


def reset_name_counters() -> None:
    _counters["func"] = 0
    _counters["tensor"] = 0


def _safe(name: str) -> str:
    name = re.sub(r"[^0-9a-zA-Z_]", "_", name)
    return name if not name[:1].isdigit() else "_" + name


def name_graph(sorted_graph: List[Tensor]) -> None:
    used = set()
    for t in sorted_graph:
        if t._attrs["name"] is not None:
            orig = t._attrs["name"]
            safe = _safe(orig)
            if safe != orig and t._attrs["original_name"] is None:
                t._attrs["original_name"] = orig
            t._attrs["name"] = safe
            used.add(safe)
    for op in sorted_ops(sorted_graph):
        if op._attrs["name"] is None:
            op._attrs["name"] = f"{op._attrs['op']}_{_counters['func']}"
            _counters["func"] += 1
        else:
            op._attrs["name"] = _safe(op._attrs["name"])
    for t in sorted_graph:
        if t._attrs["name"] is None:
            src = list(t._attrs["src_ops"])
            if src:
                op = src[0]
                idx = [id(o) for o in op._attrs["outputs"]].index(id(t))
                name = f"{op._attrs['name']}_{idx}"
            else:
                name = f"tensor_{_counters['tensor']}"
                _counters["tensor"] += 1
            while name in used:
                name += "_"
            t._attrs["name"] = name
            used.add(name)
    # dims: user-given names win; dims with the same symbol share one name
    by_symbol: Dict[str, str] = {}
    dim_used = set()
    for t in sorted_graph:
        for d in t._attrs["shape"]:
            if isinstance(d, IntImm):
                continue
            if d._attrs["name"] is not None:
                d._attrs["name"] = _safe(d._attrs["name"])
                by_symbol.setdefault(str(d._attrs["symbolic_value"]), d._attrs["name"])
                dim_used.add(d._attrs["name"])
    for t in sorted_graph:
        for i, d in enumerate(t._attrs["shape"]):
            if isinstance(d, IntImm) or d._attrs["name"] is not None:
                continue
            sym = str(d._attrs["symbolic_value"])
            if sym in by_symbol:
                d._attrs["name"] = by_symbol[sym]
                continue
            name = f"{t._attrs['name']}_dim_{i}"
            while name in dim_used:
                name += "_"
            d._attrs["name"] = name
            by_symbol[sym] = name
            dim_used.add(name)
