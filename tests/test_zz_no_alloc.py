"""The allocation-free GEMM entry point, b200ait_gemm_rcr_static_scratch.

Some callers of this library cannot call cudaMalloc: a server that carved up the device at start-up,
a host framework whose allocator owns all device memory, code that must keep driver allocation calls
off its path. For them the library offers one GEMM entry point whose split-K scratch and status
word sit in a static device array. This test drives it through the C ABI next to the ordinary entry
point (which gets a torch-allocated workspace) and requires the same results, on two calls in a
row so that what the first call left in the shared scratch cannot leak into the second. The file
name sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-2  # the tolerance of the other GEMM tests


def _rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).half().cuda()


def _call_static(lib, x, w, b, d0, out, epilogue, status):
    m, k = x.shape
    n = w.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    return lib.b200ait_gemm_rcr_static_scratch(
        x.data_ptr(), w.data_ptr(), b.data_ptr(), d0.data_ptr() if d0 is not None else None, None, out.data_ptr(),
        1, m, n, k, k, k, n, n, 0, 0, 0, 0, epilogue, 1, ctypes.c_float(1.0), 0, 1, 1, 1, 0, 0,
        status.data_ptr(), stream)


def test_static_scratch_gemm_matches_workspace_gemm_twice_in_a_row():
    from aitemplate_b200 import _lib, kernels

    lib = _lib.load()
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    # two different split-K problems back to back: the second is smaller and splits differently, so
    # stale partial sums from the first would show up in it
    cases = [((128, 768, 3072), "add", 1), ((64, 264, 2048), "fast_gelu", 2), ((128, 768, 3072), "add", 3)]
    for (m, n, k), epilogue, seed in cases:
        assert kernels.gemm_workspace_bytes(1, m, n, k) > 0, "the case is meant to exercise split-K"
        x, w, b = _rand((m, k), seed), _rand((n, k), seed + 10, 0.05), _rand((n,), seed + 20)
        d0 = _rand((m, n), seed + 30) if epilogue == "add" else None
        want = kernels.gemm_rcr(x, w, b, d0, epilogue=epilogue)  # existing entry point, torch-allocated workspace
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        code = _call_static(lib, x, w, b, d0, got, kernels.epilogue_code(epilogue), status)
        assert code == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        err = (got.float() - want.float()).abs()
        assert bool((err <= TOL + TOL * want.float().abs()).all()), f"max abs err {float(err.max()):.4g}"


def test_static_scratch_gemm_rejects_problems_beyond_its_limit():
    from aitemplate_b200 import _lib

    lib = _lib.load()
    m, n, k = 2048, 2048, 64  # 2 * m * n * 4 bytes = 32 MiB > 16 MiB
    x, w, b = _rand((m, k), 1), _rand((n, k), 2), _rand((n,), 3)
    out = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    assert _call_static(lib, x, w, b, None, out, 0, status) != 0
    msg = _lib.last_error()
    assert "too large for the static scratch" in msg and "16777216" in msg
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0  # nothing ran
