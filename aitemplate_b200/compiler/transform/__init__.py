"""Graph passes needed to execute a graph on the native runtime: toposort, parameter marking,
naming, elementwise/GEMM fusion, strided-output fusion into concatenate, memory planning. The reference's remaining ~25 optimisation passes
(python/aitemplate/compiler/transform/optimize_graph.py:104-143) are outside the hot path."""
from .fuse_mm_elementwise import fuse_mm_elementwise  # noqa: F401
from .memory_planning import memory_planning  # noqa: F401
from .name_graph import name_graph, reset_name_counters  # noqa: F401
from .toposort import mark_param_tensor, remove_no_ops, split_to_views, toposort  # noqa: F401
from .transform_strided_ops import (  # noqa: F401
    fuse_gemm_permute0213,
    fuse_permute_into_attention,
    fuse_split_strided,
    fuse_strided_cat,
)
