"""The allocation-free GEMM entry point, b200ait_gemm_rcr_static_scratch.

Some callers of this library cannot call cudaMalloc: a server that carved up the device at start-up,
a host framework whose allocator owns all device memory, code that must keep driver allocation calls
off its path. For them the library offers one GEMM entry point whose split-K scratch and status
word sit in a static device array. This test drives it through the C ABI next to the ordinary entry
point (which gets a torch-allocated workspace) and requires the same results, on two calls in a
row so that what the first call left in the shared scratch cannot leak into the second; both are
also held to the CPU oracle, and a further test checks that free device memory does not move
across calls. The file
name sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu

TOL = 1e-2  # the tolerance of the other GEMM tests


def _rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).half().cuda()


def _call_static(lib, x, w, b, d0, out, epilogue, status, dims=None):
    """x [M, K] or [B, M, K] (then w is [B, N, K]); status may be None (a null status_out)."""
    batch = x.shape[0] if x.dim() == 3 else 1
    m, k = x.shape[-2:]
    n = w.shape[-2]
    if dims is not None:
        batch, m, n, k = dims
    stream = torch.cuda.current_stream().cuda_stream
    return lib.b200ait_gemm_rcr_static_scratch(
        x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
        d0.data_ptr() if d0 is not None else None, None, out.data_ptr(),
        batch, m, n, k, k, k, n, n, m * k, n * k, m * n, m * n, epilogue, 1, ctypes.c_float(1.0), 0, 1, 1, 1, 0, 0,
        status.data_ptr() if status is not None else None, stream)


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
        ref = oracle.gemm_rcr(x, w, b, d0, epilogue=epilogue)  # and against the CPU oracle
        err = (got.float().cpu() - ref).abs()
        assert bool((err <= TOL + TOL * ref.abs()).all()), f"max abs err vs oracle {float(err.max()):.4g}"


def test_static_scratch_gemm_batched_null_status_and_no_allocation():
    from aitemplate_b200 import _lib, kernels

    lib = _lib.load()
    a, b = _rand((6, 96, 1536), 40), _rand((6, 200, 1536), 41, 0.05)  # batched (bmm_rcr form), deep K
    want = oracle.bmm_rcr(a, b)
    got = torch.full((6, 96, 200), float("nan"), dtype=torch.float16, device="cuda")
    assert _call_static(lib, a, b, None, None, got, 0, None) == 0, _lib.last_error()  # warm call, null status_out
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):
        got.fill_(float("nan"))
        assert _call_static(lib, a, b, None, None, got, 0, None) == 0, _lib.last_error()
        torch.cuda.synchronize()
        err = (got.float().cpu() - want).abs()
        assert bool((err <= TOL + TOL * want.abs()).all()), f"max abs err {float(err.max()):.4g}"
    assert torch.cuda.mem_get_info()[0] == free_before, "the entry point must not allocate device memory"
    assert kernels.device_status() == 0


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
    # dimensions whose byte count does not fit 64 bits must be rejected too, not wrap around the check
    assert _call_static(lib, x, w, b, None, out, 0, status, dims=(1 << 20, 1 << 22, 1 << 22, 64)) != 0
    assert "too large for the static scratch" in _lib.last_error()
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0  # nothing ran
