"""Compile-time GEMM profiling: picks the tile width / split-K of every gemm_rcr-family op by timing the
candidates on the GPU, the way the reference's `profile` pass picks a CUTLASS instance per op and problem
size (python/aitemplate/compiler/transform/profile.py, ops/gemm_universal/gemm_common.py:579-935), with the
winners kept in a cache file (backend/profiler_cache.py). Without profiling the library's own planner
chooses at launch; profiling only overrides it with a measured choice.

Dynamic M: one size is profiled per op, chosen by the DynamicProfileStrategy as in the reference (MAX: upper
bound, MIN: lower bound); the choice applies to the whole range.
"""
from __future__ import annotations

import logging
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..base import IntImm, Tensor
from .toposort import sorted_ops

_LOGGER = logging.getLogger(__name__)

# (tile_n, split_k); split_k 1 = never split, n = at most n splits
# (tile_n, split_k); (0, 0) is the library's own plan, which also reaches the weight-streaming kernels (few rows or few tiles)
CANDIDATES: Sequence[Tuple[int, int]] = ((0, 0), (64, 1), (128, 1), (256, 1), (512, 1), (128, 2), (256, 2),
                                         (256, 4), (128, 4), (256, 8))


def _problem_of(op, use_max: bool) -> Optional[Tuple[int, int, int]]:
    a, b = op._attrs["inputs"][0], op._attrs["inputs"][1]
    bs, as_ = b._attrs["shape"], a._attrs["shape"]
    if not (isinstance(bs[0], IntImm) and isinstance(as_[-1], IntImm)):
        return None
    m = 1
    for d in as_[:-1]:
        m *= d.upper_bound() if use_max else d.lower_bound()
    return int(m), int(bs[0].value()), int(as_[-1].value())


def profile_gemms(sorted_graph: List[Tensor], cache, timer: Optional[Callable] = None, use_max: bool = True,
                  device_name: str = "") -> Dict[str, Tuple[int, int]]:
    """Sets `tile_n` / `split_k` on every gemm op from the cache, timing the candidates with `timer` on a miss
    (timer(op, m, n, k, tile_n, split_k) -> microseconds, or None when that configuration is not legal).
    With timer None only cached choices are applied. Returns {op name: (tile_n, split_k)}."""
    from ...backend.profiler_cache import gemm_key
    from ..ops.gemm_universal.gemm_rcr import gemm

    chosen: Dict[str, Tuple[int, int]] = {}
    dirty = False
    for op in sorted_ops(sorted_graph):
        if not isinstance(op, gemm):
            continue
        prob = _problem_of(op, use_max)
        if prob is None or 0 in prob:
            continue
        m, n, k = prob
        key = gemm_key(op._attrs["op"], op._attrs["inputs"][0].dtype(), m, n, k, op._attrs.get("layout") or "",
                       device_name)
        best = cache.lookup(key)
        if best is None and timer is not None:
            timings = []
            for tile_n, split_k in CANDIDATES:
                us = timer(op, m, n, k, tile_n, split_k)
                if us is not None:
                    timings.append((us, tile_n, split_k))
            if timings:
                us, tile_n, split_k = min(timings)
                cache.insert(key, tile_n, split_k, us)
                dirty = True
                best = (tile_n, split_k)
                _LOGGER.info("profiled %s %dx%dx%d: tile_n=%d split_k=%d %.1f us", op._attrs["op"], m, n, k, tile_n,
                             split_k, us)
        if best is not None:
            op._attrs["tile_n"], op._attrs["split_k"] = best
            op._attrs["profiled"] = True
            chosen[op._attrs["name"] or op._attrs["op"]] = best
    if dirty:
        cache.save()
    return chosen


def cuda_gemm_timer(op, m: int, n: int, k: int, tile_n: int, split_k: int) -> Optional[float]:
    """Times one configuration of the op's GEMM on the current CUDA device with synthetic operands: a CUDA graph
    of launches over three operand sets (so that no launch finds its inputs in L2), best of three replays."""
    import torch

    from ... import kernels as K

    dtype = torch.float16 if op._attrs["inputs"][0].dtype() == "float16" else torch.bfloat16
    epilogue = op._attrs["op"].replace("gemm_rcr_bias", "").replace("gemm_rcr", "").lstrip("_")
    layout = op._attrs.get("layout")
    permute, playout = None, "20314"
    if layout == "Permute5D_20314":
        permute, epilogue = tuple(op._attrs["shape"]), ""
    elif layout == "Permute4D_0213":
        permute, playout, epilogue = tuple(op._attrs["shape"]), "0213", ""
    nres = int(op._attrs.get("num_sources", 0))
    sets = 3
    try:
        xs = [torch.randn((m, k), device="cuda").to(dtype) for _ in range(sets)]
        w = (torch.randn((n, k), device="cuda") * 0.02).to(dtype)
        b = torch.randn((n,), device="cuda").to(dtype) if "bias" in op._attrs["op"] else None
        ds = [torch.randn((m, n), device="cuda").to(dtype) for _ in range(nres)]
        outs = [K.gemm_rcr(xs[0], w, b, *ds, epilogue=epilogue, permute_shape=permute, permute_layout=playout,
                           tile_n=tile_n, split_k=split_k) for _ in range(sets)]

        def launch(i: int) -> None:
            K.gemm_rcr(xs[i % sets], w, b, *ds, epilogue=epilogue, permute_shape=permute, permute_layout=playout,
                       tile_n=tile_n, split_k=split_k, out=outs[i % sets])

        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        reps = 6
        with torch.cuda.stream(side):
            launch(0)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    launch(i)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / reps)
        return best * 1e3
    except (RuntimeError, ValueError) as e:  # configuration not legal for this problem
        _LOGGER.debug("candidate tile_n=%d split_k=%d rejected: %s", tile_n, split_k, e)
        return None
