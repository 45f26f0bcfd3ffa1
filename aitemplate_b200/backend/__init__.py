"""Backend: the single CUDA sm_100a target (kernels are prebuilt in libb200ait.so)."""
from . import target  # noqa: F401
