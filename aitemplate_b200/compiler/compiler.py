"""compile_model(): graph -> executable plan -> Model.

Same signature and validation as the reference (python/aitemplate/compiler/compiler.py:149-354), but
where the reference renders C++ per op, runs nvcc and links `test.so`, this build lowers the graph to
a *plan* for the prebuilt runtime in libb200ait.so:

  toposort -> remove_no_ops -> mark_param_tensor -> fuse_mm_elementwise -> fuse_gemm_permute0213 -> fuse_permute_into_attention -> split_to_views
  -> fuse_split_strided -> fuse_strided_cat -> name_graph
  -> memory_planning -> write <workdir>/<test_name>/<dll_name>.plan (+ constants.bin) -> Model(plan)

There is no code generation. Profiling is optional: by default the library's planner picks tile width and
split-K at launch; with `profile_devs` given (or AIT_B200_PROFILE=1) every gemm_rcr-family op is timed over
the launch configurations on the current GPU, per `dynamic_profiling_strategy` for dynamic M, and the winners
are written into the plan and kept in a cache file (`profile_dir`, default ~/.aitemplate_b200).
`profile_timeout` and `debug_settings` are accepted for compatibility and ignored.
"""
from __future__ import annotations

import logging
import os
from typing import Dict, List, Optional, Union

from .base import DynamicProfileStrategy, IntImm, Tensor
from .dtype import dtype_str_to_enum
from .model import Model
from .transform import (
    fuse_mm_elementwise,
    fuse_gemm_permute0213,
    fuse_permute_into_attention,
    fuse_split_strided,
    fuse_strided_cat,
    mark_param_tensor,
    memory_planning,
    name_graph,
    remove_no_ops,
    reset_name_counters,
    split_to_views,
    toposort,
)
from .transform.memory_planning import storage_root
from .transform.toposort import sorted_ops

_LOGGER = logging.getLogger(__name__)

KIND_INPUT, KIND_OUTPUT, KIND_CONSTANT, KIND_BLOB, KIND_VIEW = range(5)


def _validate_tensor_args(sorted_graph: List[Tensor], output_tensors: List[Tensor]) -> None:
    """Errors on duplicate names, non-outputs in the list, or reachable outputs missing from it
    (python/aitemplate/compiler/compiler.py:50-76)."""
    seen = set()
    for t in output_tensors:
        name = t._attrs["name"]
        if not t._attrs["is_output"]:
            raise ValueError(f"Got non-output tensor in output_tensors list: {name}")
        if name in seen:
            raise ValueError(f"Got duplicate name {name} in output_tensors list.")
        seen.add(name)
    for t in reversed(sorted_graph):
        if t._attrs["is_output"] and t._attrs["name"] not in seen:
            raise ValueError(f"Output {t._attrs['name']} was not passed into output_tensors")


def _assign_storage(sorted_graph: List[Tensor], outputs: List[Tensor]):
    """Decides where every tensor lives. Returns the list of (src, dst) copies needed for outputs
    that alias an input, a constant or another output (static/include/model_container.h:127-130)."""
    copies = []
    claimed = {}
    for slot, out in enumerate(outputs):
        root = storage_root(out)
        external = root._attrs["is_input"] or root._attrs["is_param"] or id(root) in claimed
        if external and root is not out:
            # the output is a view of storage it cannot take over: give it its own buffer + a copy
            out._attrs["own_output_slot"] = slot
            copies.append(out)
        elif external:
            raise ValueError(f"Output {out._attrs['name']} is an input or a constant of the model")
        else:
            root._attrs["output_slot"] = slot
            claimed[id(root)] = slot
    return copies


def _lower_to_plan(sorted_graph: List[Tensor], outputs: List[Tensor], test_name: str, blob_bytes: int,
                   constants_bytes: int, copies: List[Tensor], constants_file: Optional[str], bound: Dict[str, tuple]) -> str:
    dims: Dict[str, int] = {}
    dim_lines: List[str] = []

    def tok(d) -> str:
        if isinstance(d, IntImm):
            return f"s{d.value()}"
        name = d._attrs["name"]
        if name not in dims:
            dims[name] = len(dims)
            dim_lines.append(f"dim {name} {d.lower_bound()} {d.upper_bound()}")
        return f"d{dims[name]}"

    index: Dict[int, int] = {}
    tensor_lines: List[str] = []
    input_slots: List[int] = []

    def emit(t: Tensor, kind: int, slot: int, offset: int, base: int, name: Optional[str] = None) -> int:
        idx = len(tensor_lines)
        shape = " ".join(tok(d) for d in t._attrs["shape"])
        tensor_lines.append(
            f"tensor {name or t._attrs['name']} {dtype_str_to_enum(t.dtype())} {kind} {slot} {offset} {base} "
            f"{len(t._attrs['shape'])} {shape}".rstrip())
        return idx

    # inputs first (their dims bind the dynamic-dim table), in graph order
    for t in sorted_graph:
        if t._attrs["is_input"] and t._attrs["is_view_of"] is None:
            index[id(t)] = emit(t, KIND_INPUT, len(input_slots), 0, -1)
            input_slots.append(index[id(t)])
    def place(t: Tensor) -> None:
        if id(t) in index or t.is_a_const_num():
            return
        view_of = t._attrs["is_view_of"]
        if view_of is not None:
            place(view_of)  # the runtime wants a base before its views (a producer fused into a concat
            # aliases the concat output, which comes later in graph order)
            alias = t._attrs["name"] + "__alias" if t._attrs.get("own_output_slot") is not None else None
            index[id(t)] = emit(t, KIND_VIEW, -1, t._attrs.get("view_offset_bytes", 0), index[id(view_of)], name=alias)
        elif t._attrs["is_param"]:
            index[id(t)] = emit(t, KIND_CONSTANT, -1, t._attrs["offset"], -1)
        elif t._attrs.get("output_slot") is not None:
            index[id(t)] = emit(t, KIND_OUTPUT, t._attrs["output_slot"], 0, -1)
        else:
            index[id(t)] = emit(t, KIND_BLOB, -1, t._attrs["offset"], -1)

    for t in sorted_graph:
        place(t)
    op_lines: List[str] = []

    def op_line(kernel: str, name: str, operands, outs, ints, floats) -> None:
        parts = ["op", kernel, name, str(len(operands))] + [str(o) for o in operands]
        parts += [str(len(outs))] + [str(o) for o in outs]
        parts += [str(len(ints))] + [str(int(i)) for i in ints]
        parts += [str(len(floats))] + [repr(float(f)) for f in floats]
        op_lines.append(" ".join(parts))

    for op in sorted_ops(sorted_graph):
        low = op._lower()
        outs = [index[id(o)] for o in op._attrs["outputs"]]
        kernel = low["kernel"]
        if kernel == "view":
            op_line("view", op._attrs["name"], [index[id(op._attrs["inputs"][0])]], outs, [], [])
        elif kernel == "elementwise":
            operands = [index[id(x)] for x in low["inputs"]]
            ints = [len(low["steps"])]
            floats = []
            for code, operand, const in low["steps"]:
                ints += [code, operand]
                floats.append(const)
            op_line("elementwise", op._attrs["name"], operands, outs, ints, floats)
        else:
            operands = [index[id(x)] if x is not None else -1 for x in low["operands"]]
            op_line(kernel, op._attrs["name"], operands, outs, low["ints"], low["floats"])
    # outputs that alias external storage: own buffer + device copy
    output_slots: Dict[int, int] = {}
    for slot, out in enumerate(outputs):
        if out._attrs.get("own_output_slot") is not None:
            idx = emit(out, KIND_OUTPUT, slot, 0, -1)
            op_line("copy", f"copy_{out._attrs['name']}", [index[id(out)]], [idx], [], [])
            output_slots[slot] = idx
        else:
            output_slots[slot] = index[id(out)]
    const_lines = []
    for t in sorted_graph:
        if t._attrs["is_param"] and t._attrs["is_view_of"] is None:
            name = t._attrs["name"]
            is_bound, file_off = bound.get(name, (False, 0))
            const_lines.append(
                f"constant {name} {t._attrs['original_name'] or name} {index[id(t)]} {t._attrs['offset']} "
                f"{t.size_bytes()} {1 if is_bound else 0} {file_off}")
    # a user-visible output may be a view of the tensor that owns the output buffer; the runtime
    # reports name / dtype / shape of the user-visible one
    lines = [
        "B200AIT_PLAN 1", f"name {test_name}", f"blob_bytes {blob_bytes}", f"constants_bytes {constants_bytes}",
        f"constants_file {constants_file or '-'}", f"num_dims {len(dim_lines)}", *dim_lines,
        f"num_tensors {len(tensor_lines)}", *tensor_lines, f"num_ops {len(op_lines)}", *op_lines,
        f"num_constants {len(const_lines)}", *const_lines,
        f"num_inputs {len(input_slots)}", *[f"input {i} {t}" for i, t in enumerate(input_slots)],
        f"num_outputs {len(outputs)}", *[f"output {s} {output_slots[s]}" for s in range(len(outputs))],
    ]
    return "\n".join(lines) + "\n"


def _profile(graph: List[Tensor], profile_dir: Optional[str], strategy) -> None:
    """Compile-time GEMM profiling (python/aitemplate/compiler/compiler.py:286-306 in the reference)."""
    from ..backend.profiler_cache import GemmProfileCache
    from .transform.profile import cuda_gemm_timer, profile_gemms

    cache = GemmProfileCache(os.path.join(profile_dir, "gemm_profile_cache.json") if profile_dir else None)
    timer, device = None, ""
    try:
        import torch

        if torch.cuda.is_available():
            timer, device = cuda_gemm_timer, torch.cuda.get_device_name()
    except ImportError:
        pass
    if timer is None:
        _LOGGER.warning("no CUDA device: only cached GEMM profiles are applied")
    profile_gemms(graph, cache, timer, use_max=strategy != DynamicProfileStrategy.MIN, device_name=device)


def compile_model(
    tensor: Union[Tensor, List[Tensor]],
    target,
    workdir: str,
    test_name: str,
    profile_devs: List[int] = None,
    dynamic_profiling_strategy: DynamicProfileStrategy = DynamicProfileStrategy.MAX,
    dll_name: str = "test.so",
    num_runtimes: int = 1,
    profile_dir: str = None,
    constants: Optional[Dict[str, object]] = None,
    allocator_kind=None,
    debug_settings=None,
    do_optimize_graph: bool = True,
    profile_timeout: int = 500,
) -> Model:
    """Compiles the graph that ends in `tensor` (one output or a list; output order = list order)
    and returns a Model bound to it. `constants` maps constant names to torch / numpy tensors whose
    bytes are stored with the model; other constants must be set on the Model before the first run."""
    if constants is None:
        constants = {}
    test_name = test_name.replace(",", "_")
    test_dir = os.path.join(workdir, test_name)
    plan_path = os.path.join(test_dir, dll_name + ".plan")
    recompile = os.getenv("AIT_RECOMPILE", "1")
    if int(recompile) == 0:
        return Model(plan_path, num_runtimes, allocator_kind)
    os.makedirs(test_dir, exist_ok=True)
    outputs = [tensor] if isinstance(tensor, Tensor) else list(tensor)
    reset_name_counters()
    graph = toposort(outputs)
    _validate_tensor_args(graph, outputs)
    # bind constants by name before anything renames tensors (transform/bind_constants.py:26-54)
    by_name = {t._attrs["name"]: t for t in graph if t._attrs["name"] is not None}
    for name, data in constants.items():
        if name not in by_name:
            _LOGGER.warning("constant %s is not used by the graph", name)
            continue
        t = by_name[name]
        if t._attrs["is_input"]:
            raise ValueError(f"Cannot bind input tensor {name}")
        t._bind_data(data)
    graph = remove_no_ops(graph)
    mark_param_tensor(graph)
    if do_optimize_graph:
        graph = fuse_mm_elementwise(graph, outputs)
        graph = fuse_gemm_permute0213(graph, outputs)
        graph = fuse_permute_into_attention(graph, outputs)
        mark_param_tensor(graph)
        split_to_views(graph)
        fuse_split_strided(graph)
        fuse_strided_cat(graph)
    name_graph(graph)
    if profile_devs is not None or os.getenv("AIT_B200_PROFILE", "0") == "1":
        _profile(graph, profile_dir, dynamic_profiling_strategy)
    copies = _assign_storage(graph, outputs)
    blob_bytes, constants_bytes = memory_planning(graph)
    bound: Dict[str, tuple] = {}
    constants_file = None
    blobs = []
    file_off = 0
    for t in graph:
        if t._attrs["is_param"] and t._attrs["data"] is not None:
            raw = t._attrs["data"].to_bytes()
            bound[t._attrs["name"]] = (True, file_off)
            blobs.append(raw)
            file_off += len(raw)
    if blobs:
        constants_file = "constants.bin"
        with open(os.path.join(test_dir, constants_file), "wb") as f:
            for raw in blobs:
                f.write(raw)
    plan = _lower_to_plan(graph, outputs, test_name, blob_bytes, constants_bytes, copies, constants_file, bound)
    with open(plan_path, "w") as f:
        f.write(plan)
    module = Model(plan_path, num_runtimes, allocator_kind)
    module.debug_sorted_graph = graph
    return module
