"""detect_target(): returns the CUDA sm_100a target.

The reference probes nvidia-smi / the driver and maps compute capability >= 9.0 to "90"
(python/aitemplate/testing/detect_target.py:68-133). This build has one target; the probe only
verifies, when a GPU is visible, that it is a compute-capability 10.x device.
"""
from __future__ import annotations

from ..backend.target import CUDA

_FLAG = None


def detect_target(**kwargs) -> CUDA:
    global _FLAG
    if _FLAG is None:
        try:
            import torch

            if torch.cuda.is_available():
                major, _ = torch.cuda.get_device_capability()
                if major != 10:
                    raise RuntimeError(
                        f"aitemplate_b200 needs an sm_100a GPU (B200); found compute capability {major}.x")
        except ImportError:  # pragma: no cover
            pass
        _FLAG = "100"
    return CUDA(arch=_FLAG, **kwargs)
