"""Testing helpers mirroring python/aitemplate/testing: detect_target, random tensors, benchmarks."""
from . import benchmark_pt, test_utils  # noqa: F401
from .detect_target import detect_target  # noqa: F401
