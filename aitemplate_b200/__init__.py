"""aitemplate_b200: a B200-native (sm_100a) implementation of AITemplate's fused-GEMM hot path
behind the reference's graph-node / compile_model() / Model.run_with_tensors() API."""

__version__ = "0.1.0"
