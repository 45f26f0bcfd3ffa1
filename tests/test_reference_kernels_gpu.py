"""Compares this repository's softmax and permute kernels with the REFERENCE's own CUDA kernels on
the same device buffers.

oracle/_ref/libref_kernels.so is the reference's softmax.cuh and permute.cuh compiled for sm_100a by
oracle/build_ref.py (entry points in oracle/ref_kernels.cu, which holds no kernel code of its own).
It is built where a reference checkout exists and travels with the tree as a built file; without it
these tests skip. permute must agree bit for bit; softmax, which both sides evaluate in fp32 and
round once to fp16, within one fp16 unit in the last place (at most 2^-10 relative, 2^-24 absolute for subnormals),
and both within the reference's own tolerance (1e-2) of the CPU oracle.
"""
import ctypes
import os

import pytest
import torch

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu

_REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                        "libref_kernels.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(_REF_LIB):
        pytest.skip("oracle/_ref/libref_kernels.so not built (needs a reference checkout at build time)")
    lib = ctypes.CDLL(_REF_LIB)
    lib.ref_softmax_half.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
    lib.ref_softmax_half.restype = ctypes.c_int
    lib.ref_permute_half.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int64),
                                     ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]
    lib.ref_permute_half.restype = ctypes.c_int
    return lib


def _rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).half()


@pytest.mark.parametrize("k", [64, 128, 384, 1024, 4096, 77])
@pytest.mark.parametrize("m", [1, 333, 4096])
def test_softmax_matches_reference_kernel(ref, m, k):
    from aitemplate_b200 import kernels

    x = _rand((m, k), 100 + k, scale=2.0)
    xd = x.cuda()
    want = torch.empty_like(xd)
    rc = ref.ref_softmax_half(xd.data_ptr(), want.data_ptr(), m, k, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    got = kernels.softmax(xd, dim=-1)
    torch.cuda.synchronize()
    g, w = got.float().cpu(), want.float().cpu()
    err = (g - w).abs()
    assert bool((err <= 2.0 ** -10 * torch.maximum(w, g) + 2.0 ** -24).all()), float(err.max())
    o = oracle.softmax(x, -1)
    for t in (g, w):
        assert bool(((t - o).abs() <= 1e-2 + 1e-2 * o).all())


@pytest.mark.parametrize("shape,dims", [
    ((2, 4096, 8, 40), (0, 2, 1, 3)),
    ((64, 384, 12, 64), (0, 2, 1, 3)),
    ((3, 5, 7), (0, 2, 1)), ((3, 5, 7), (1, 0, 2)), ((3, 5, 7), (2, 1, 0)),
    ((33, 129, 66), (2, 0, 1)),
    ((4, 3, 4, 5, 6), (4, 0, 3, 1, 2)),
    ((2, 8, 3, 4, 16), (2, 0, 3, 1, 4)),
])
def test_permute_matches_reference_kernel_bitwise(ref, shape, dims):
    from aitemplate_b200 import kernels

    x = _rand(shape, 7).cuda()
    want = torch.empty([shape[d] for d in dims], dtype=torch.float16, device="cuda")
    c_dims = (ctypes.c_int64 * len(shape))(*shape)
    c_perm = (ctypes.c_int * len(dims))(*dims)
    rc = ref.ref_permute_half(want.data_ptr(), x.data_ptr(), len(shape), c_dims, c_perm,
                              torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    got = kernels.permute(x, dims)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert torch.equal(got.cpu(), oracle.permute(x, dims))
