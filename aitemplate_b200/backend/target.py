"""Target: the compilation target handed to compile_model().

The reference's Target (python/aitemplate/backend/target.py:54-347, cuda/target_def.py:146-280) selects an
nvcc arch among {70, 75, 80, 90}, builds the CUTLASS generator and carries feature flags as kwargs.
Here there is exactly one target, CUDA sm_100a with prebuilt kernels; kwargs are kept in `_kwargs` so
code that reads `Target.current()._kwargs` keeps working. `use_fp16_acc=True` is rejected: every
contraction accumulates in fp32.
"""
from __future__ import annotations

from typing import Optional

CURRENT_TARGET: Optional["Target"] = None


class Target:
    def __init__(self, arch: str = "100", **kwargs) -> None:
        if kwargs.get("use_fp16_acc", False):
            raise NotImplementedError("use_fp16_acc=True is not supported: the sm_100a kernels accumulate in fp32")
        self._arch = str(arch)
        self._kwargs = dict(kwargs)
        self._target_type = 1

    def name(self) -> str:
        return "cuda"

    def arch(self) -> str:
        return self._arch

    def __enter__(self):
        global CURRENT_TARGET
        self._prev = CURRENT_TARGET
        CURRENT_TARGET = self
        return self

    def __exit__(self, *args) -> None:
        global CURRENT_TARGET
        CURRENT_TARGET = getattr(self, "_prev", None)

    @staticmethod
    def current() -> "Target":
        if CURRENT_TARGET is None:
            raise RuntimeError("Target has not been initialized.")
        return CURRENT_TARGET

    def use_dummy_profiling_results(self) -> bool:
        return True  # nothing is profiled at compile time


class CUDA(Target):
    """CUDA target; only arch "100" (B200, sm_100a) exists in this build."""

    def __init__(self, arch: str = "100", **kwargs) -> None:
        if str(arch) not in ("100", "100a"):
            raise RuntimeError(f"Unsupported CUDA architecture {arch}: this build targets sm_100a only")
        super().__init__("100", **kwargs)
