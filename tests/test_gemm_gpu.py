"""GPU parity of the gemm_rcr / bmm_rcr family against the CPU oracle, through the C ABI.

Shapes follow the reference's tests: tests/unittest/ops/test_gemm_bias.py:43-99 (M 4096/1000, (N,K) in
{(4,4),(81,1024),(3,256),(64,1024)}, zero sizes), test_gemm_rcr_bias_fast_gelu.py:44-128 (M in
{1,7,64,127,128}, K=1024, N=64), test_gemm_bias_broadcast.py (8x8x8, 256x128, 1024x512),
test_bmm.py:32-70, plus the benchmark configurations.
Tolerance: atol = rtol = 1e-2 against the fp32 oracle (fp16 storage, fp32 accumulation).
"""
import pytest
import torch

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu

ATOL = RTOL = 1e-2


def _kernels():
    from aitemplate_b200 import kernels

    return kernels


def _rand(shape, seed, dist="normal", scale=1.0, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    if dist == "uniform":
        t = torch.rand(shape, generator=g) * 2 - 1
    else:
        t = torch.randn(shape, generator=g)
    return (t * scale).to(dtype)


def _close(got, want, atol=ATOL, rtol=RTOL):
    got = got.float().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all()
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    bad = err > bound
    assert not bad.any(), (
        f"{int(bad.sum())}/{bad.numel()} mismatches, max abs err {float(err.max()):.4g}, "
        f"first bad index {bad.nonzero()[0].tolist()}"
    )


def test_config1_gemm_rcr_bias_fast_gelu():
    k = _kernels()
    x = _rand((256, 768), 1234, "uniform")
    w = _rand((3072, 768), 1235, scale=0.02)
    b = _rand((3072,), 1236, scale=0.02)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), epilogue="fast_gelu")
    _close(y, oracle.gemm_rcr(x, w, b, epilogue="fast_gelu"))


@pytest.mark.parametrize("epilogue", sorted(oracle.EPILOGUES.keys()))
def test_every_epilogue(epilogue):
    k = _kernels()
    m, n, kk = 384, 520, 256
    x = _rand((m, kk), 1, "uniform")
    w = _rand((n, kk), 2, scale=0.05)
    b = _rand((n,), 3, scale=0.5)
    d0 = _rand((m, n), 4)
    d1 = _rand((m, n), 5)
    _, b1, b2, _ = oracle.EPILOGUES[epilogue]
    kw = dict(epilogue=epilogue)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), d0.cuda() if b1 else None, d1.cuda() if b2 else None, **kw)
    _close(y, oracle.gemm_rcr(x, w, b, d0 if b1 else None, d1 if b2 else None, **kw))


@pytest.mark.parametrize("m", [1, 7, 64, 127, 128, 129, 1000])
@pytest.mark.parametrize("n,kk", [(64, 1024), (72, 72), (264, 8), (512, 200)])
def test_ragged_shapes(m, n, kk):
    k = _kernels()
    x = _rand((m, kk), 10 + m, "uniform")
    w = _rand((n, kk), 11 + n, scale=0.05)
    b = _rand((n,), 12, scale=0.1)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), epilogue="relu")
    _close(y, oracle.gemm_rcr(x, w, b, epilogue="relu"))


@pytest.mark.parametrize("n,kk", [(4, 4), (81, 1024), (3, 256), (64, 1021), (7, 5)])
def test_unaligned_shapes_use_cuda_core_kernel(n, kk):
    k = _kernels()
    m = 1000
    x = _rand((m, kk), 20, "uniform")
    w = _rand((n, kk), 21, scale=0.05)
    b = _rand((n,), 22, scale=0.1)
    d0 = _rand((m, n), 23)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), d0.cuda(), epilogue="add_relu")
    _close(y, oracle.gemm_rcr(x, w, b, d0, epilogue="add_relu"))


@pytest.mark.parametrize("tile_n", [64, 128, 256, 512])
def test_forced_tile_width_many_tiles(tile_n):
    # more tiles than SMs: exercises the persistent loop, both accumulators and every stage phase
    k = _kernels()
    m, n, kk = 4096, 2304, 768
    x = _rand((m, kk), 30)
    w = _rand((n, kk), 31, scale=0.02)
    b = _rand((n,), 32, scale=0.02)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), epilogue="", tile_n=tile_n)
    _close(y, oracle.gemm_rcr(x, w, b))


# tile_n = 512 asks for 256 x 256 tiles computed by CTA pairs (cta_group::2); the library picks it by itself
# for large problems, these cases force it on shapes that exercise its edges.
@pytest.mark.parametrize(
    "m,n,kk,epilogue",
    [
        (256, 256, 64, ""),          # one tile, one k-block
        (512, 512, 256, "relu"),
        (200, 296, 128, ""),         # the second CTA of the pair owns rows 128..199 only; ragged N
        (100, 256, 128, "gelu"),     # the second CTA's rows are all out of range
        (200, 296, 128, "add"),      # residual boxes clipped in both directions
        (100, 256, 128, "add_relu"),
        (1000, 776, 256, "mul"),
        (2048, 1024, 512, "add"),
        (2048, 1024, 512, "add_add"),  # second residual: register path next to the staged first one
        (4096, 768, 3072, "add"),    # many tiles per pair: every ring stage and both accumulators wrap
        (512, 512, 256, "fast_gelu"),
        (4096, 3072, 768, "fast_gelu"),  # the lean pair fast_gelu kernel of the BERT FFN1 launch
        (300, 520, 192, "fast_gelu"),
    ],
)
def test_cta_pair_tiles(m, n, kk, epilogue):
    k = _kernels()
    x = _rand((m, kk), 300, dist="uniform")
    w = _rand((n, kk), 301, scale=0.05)
    b = _rand((n,), 302, scale=0.1)
    nres = {"add": 1, "add_relu": 1, "mul": 1, "add_add": 2}.get(epilogue, 0)
    d = [_rand((m, n), 303 + i) for i in range(nres)]
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue, tile_n=512)
    assert k.device_status() == 0
    _close(y, oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue))


@pytest.mark.parametrize("bsz,m,n,kk", [(3, 300, 520, 512), (8, 256, 256, 1024), (5, 128, 768, 576)])
def test_cta_pair_tiles_batched(bsz, m, n, kk):
    # bmm through the CTA-pair kernel (forced): ragged rows per batch, batch index in the TMA coordinates
    k = _kernels()
    a, b = _rand((bsz, m, kk), 330, dist="uniform"), _rand((bsz, n, kk), 331, scale=0.1)
    y = k.bmm_rcr(a.cuda(), b.cuda(), tile_n=512)
    assert k.device_status() == 0
    _close(y, oracle.bmm_rcr(a, b))
    y2 = k.bmm_rcr(a.cuda(), b.cuda(), alpha=0.125, tile_n=512)      # alpha: the generic (non-lean) pair kernel
    _close(y2, oracle.bmm_rcr(a, b, alpha=0.125))


def test_cta_pair_tiles_bf16_and_permuted_store():
    k = _kernels()
    s_, h, dd, bsz = 384, 12, 64, 4
    x = _rand((bsz * s_, h * dd), 310)
    w = _rand((3 * h * dd, h * dd), 311, scale=0.05)
    b = _rand((3 * h * dd,), 312, scale=0.1)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), permute_shape=(s_, 3, h), tile_n=512)
    _close(y, oracle.gemm_rcr_bias_permute(x, w, b, (s_, 3, h)))
    xb, wb, bb = x.to(torch.bfloat16), w.to(torch.bfloat16), b.to(torch.bfloat16)
    db = _rand((bsz * s_, 3 * h * dd), 313, dtype=torch.bfloat16)
    yb = k.gemm_rcr(xb.cuda(), wb.cuda(), bb.cuda(), db.cuda(), epilogue="add", tile_n=512)
    _close(yb, oracle.gemm_rcr(xb, wb, bb, db, epilogue="add"), atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("m,n,kk,epilogue,num_out", [(1024, 768, 512, "relu", 2), (300, 264, 128, "add", 3),
                                                      (4096, 1024, 1024, "", 8)])
def test_multi_destination_store(m, n, kk, epilogue, num_out):
    # the N-split exchange form: every tile is TMA-stored into several buffers of a wider row-major matrix
    # (here all on this GPU; on several GPUs the extra pointers are peer mappings)
    k = _kernels()
    x = _rand((m, kk), 320, dist="uniform")
    w = _rand((n, kk), 321, scale=0.05)
    b = _rand((n,), 322, scale=0.1)
    d0 = _rand((m, n), 323) if epilogue == "add" else None
    ldc, col0 = 2 * n + 64, 64
    bufs = [torch.full((m, ldc), 7.0, dtype=torch.float16, device="cuda") for _ in range(num_out)]
    ptrs = [t.data_ptr() + col0 * 2 for t in bufs]
    k.gemm_rcr_multi_out(x.cuda(), w.cuda(), b.cuda(), ptrs, ldc, d0=None if d0 is None else d0.cuda(),
                         epilogue=epilogue)
    assert k.device_status() == 0
    want = oracle.gemm_rcr(x, w, b, *([d0] if d0 is not None else []), epilogue=epilogue)
    for t in bufs:
        _close(t[:, col0:col0 + n], want)
        assert torch.equal(t[:, col0:col0 + n], bufs[0][:, col0:col0 + n])
        assert bool((t[:, :col0] == 7.0).all()) and bool((t[:, col0 + n:] == 7.0).all())  # nothing outside the block


# row-major B ("rrr" layouts of the reference: tests/unittest/ops/test_gemm.py, test_bmm.py): W stored [K, N]
@pytest.mark.parametrize("m,n,kk,tile_n", [(256, 512, 128, 0), (1000, 264, 200, 0), (128, 64, 64, 64), (300, 640, 1024, 128),
                                            (2048, 1024, 512, 256), (4096, 768, 768, 512), (7, 72, 72, 0)])
def test_gemm_rrr(m, n, kk, tile_n):
    k = _kernels()
    x = _rand((m, kk), 400, dist="uniform")
    w = _rand((kk, n), 401, scale=0.05)
    b = _rand((n,), 402, scale=0.1)
    y = k.gemm_rrr(x.cuda(), w.cuda(), b.cuda(), tile_n=tile_n)
    assert k.device_status() == 0
    _close(y, oracle.gemm_rrr(x, w, b))
    y0 = k.gemm_rrr(x.cuda(), w.cuda(), None, epilogue="", tile_n=tile_n)
    _close(y0, oracle.gemm_rrr(x, w))


def test_gemm_rrr_unaligned_uses_cuda_core_kernel():
    k = _kernels()
    x, w = _rand((33, 21), 410), _rand((21, 19), 411, scale=0.2)   # N and K not multiples of 8
    _close(k.gemm_rrr(x.cuda(), w.cuda()), oracle.gemm_rrr(x, w))


@pytest.mark.parametrize("bsz,m,n,kk", [(4, 128, 256, 64), (3, 100, 72, 40), (16, 384, 64, 384), (1, 64, 64, 64)])
def test_bmm_rrr(bsz, m, n, kk):
    k = _kernels()
    a, b = _rand((bsz, m, kk), 420, dist="uniform"), _rand((bsz, kk, n), 421, dist="uniform")
    _close(k.bmm_rrr(a.cuda(), b.cuda()), oracle.bmm_rrr(a, b))
    b1 = _rand((1, kk, n), 422, dist="uniform")                      # broadcast B over the batch
    _close(k.bmm_rrr(a.cuda(), b1.cuda()), oracle.bmm_rrr(a, b1))


def test_no_bias_and_alpha():
    k = _kernels()
    x = _rand((300, 320), 40)
    w = _rand((320, 320), 41, scale=0.05)
    y = k.gemm_rcr(x.cuda(), w.cuda(), None, alpha=0.5)
    _close(y, oracle.gemm_rcr(x, w, None, alpha=0.5))


def test_leading_dims_fold_into_m():
    k = _kernels()
    x = _rand((2, 21, 5, 64), 42)
    w = _rand((128, 64), 43, scale=0.1)
    b = _rand((128,), 44)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda())
    assert tuple(y.shape) == (2, 21, 5, 128)
    _close(y, oracle.gemm_rcr(x, w, b))


@pytest.mark.parametrize("m,n,kk", [(0, 64, 64), (64, 0, 64), (64, 64, 0)])
def test_zero_size_launches_nothing(m, n, kk):
    k = _kernels()
    x = torch.zeros((m, kk), dtype=torch.float16, device="cuda")
    w = torch.zeros((n, kk), dtype=torch.float16, device="cuda")
    b = torch.zeros((n,), dtype=torch.float16, device="cuda")
    y = k.gemm_rcr(x, w, b)
    assert tuple(y.shape) == (m, n)


def test_null_residual_is_an_error():
    k = _kernels()
    x = _rand((64, 64), 1).cuda()
    w = _rand((64, 64), 2).cuda()
    b = _rand((64,), 3).cuda()
    with pytest.raises(RuntimeError, match="d0"):
        k.gemm_rcr(x, w, b, None, epilogue="add")


def test_bf16():
    k = _kernels()
    x = _rand((512, 256), 50, dtype=torch.bfloat16)
    w = _rand((384, 256), 51, scale=0.05, dtype=torch.bfloat16)
    b = _rand((384,), 52, scale=0.1, dtype=torch.bfloat16)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), epilogue="gelu")
    _close(y, oracle.gemm_rcr(x, w, b, epilogue="gelu"), atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("bsz,s,h,d", [(2, 8, 4, 20), (4, 384, 12, 64), (2, 100, 3, 40)])
def test_permute_20314_epilogue(bsz, s, h, d):
    # the QKV projection of nn.MultiheadAttention: shape=(seq, 3, heads)
    # (python/aitemplate/frontend/nn/attention.py:162-168, tests/unittest/ops/test_attention.py:352-424)
    k = _kernels()
    hid = h * d
    x = _rand((bsz * s, hid), 60)
    w = _rand((3 * hid, hid), 61, scale=0.05)
    b = _rand((3 * hid,), 62, scale=0.1)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), permute_shape=(s, 3, h))
    assert tuple(y.shape) == (3, bsz, h, s, d)
    _close(y, oracle.gemm_rcr_bias_permute(x, w, b, (s, 3, h)))


def test_permute_0213_epilogue():
    k = _kernels()
    x = _rand((2 * 96, 320), 63)
    w = _rand((320, 320), 64, scale=0.05)
    y = k.gemm_rcr(x.cuda(), w.cuda(), None, permute_shape=(96, 8), permute_layout="0213")
    assert tuple(y.shape) == (2, 8, 96, 40)
    _close(y, oracle.gemm_rcr_bias_permute(x, w, None, (96, 8), layout="0213"))


@pytest.mark.parametrize("bsz,m,n,kk", [(1, 128, 512, 256), (5, 100, 512, 256), (64, 512, 512, 64), (3, 32, 40, 24)])
def test_bmm_rcr(bsz, m, n, kk):
    k = _kernels()
    a = _rand((bsz, m, kk), 70, "uniform")
    b = _rand((bsz, n, kk), 71, "uniform")
    y = k.bmm_rcr(a.cuda(), b.cuda())
    _close(y, oracle.bmm_rcr(a, b))


def test_bmm_rcr_broadcast_and_zero_batch():
    k = _kernels()
    a = _rand((6, 64, 128), 72, "uniform")
    b = _rand((1, 96, 128), 73, "uniform")
    _close(k.bmm_rcr(a.cuda(), b.cuda()), oracle.bmm_rcr(a, b))
    _close(k.bmm_rcr(b.cuda(), a.cuda()), oracle.bmm_rcr(b, a))
    z = k.bmm_rcr(torch.zeros((0, 8, 8), dtype=torch.float16, device="cuda"),
                  torch.zeros((0, 8, 8), dtype=torch.float16, device="cuda"))
    assert tuple(z.shape) == (0, 8, 8)


# shapes of tests/unittest/ops/test_bmm_permute.py:67-71 and :110-114 (B 24 / 100 / 10240, M 80 / 88, d1 12 / 10),
# plus tile-aligned ones that take the staged TMA store with the two-level batch coordinate
@pytest.mark.parametrize("bsz,m,n,kk,d1", [(24, 80, 64, 88, 12), (100, 88, 64, 88, 10), (10240, 88, 64, 88, 10),
                                           (48, 256, 256, 64, 12), (16, 384, 128, 128, 4), (6, 130, 200, 72, 1)])
@pytest.mark.parametrize("row_major_b", [False, True])
def test_bmm_permute(bsz, m, n, kk, d1, row_major_b):
    k = _kernels()
    a = _rand((bsz, m, kk), 90, "uniform")
    b = _rand((bsz, kk, n) if row_major_b else (bsz, n, kk), 91, "uniform")
    y = k.bmm_permute(a.cuda(), b.cuda(), d1, b_row_major=row_major_b)
    assert k.device_status() == 0
    assert tuple(y.shape) == (bsz // d1, m, d1, n)
    _close(y, oracle.bmm_permute(a, b, d1, b_row_major=row_major_b))


def test_bmm_permute_alpha_bf16_and_errors():
    k = _kernels()
    a = _rand((8, 128, 64), 92, "uniform", dtype=torch.bfloat16)
    b = _rand((8, 256, 64), 93, "uniform", dtype=torch.bfloat16)
    y = k.bmm_permute(a.cuda(), b.cuda(), 4, alpha=0.25)
    _close(y, oracle.bmm_permute(a, b, 4, alpha=0.25), atol=4e-2, rtol=4e-2)
    with pytest.raises(ValueError):
        k.bmm_permute(a.cuda(), b.cuda(), 3)           # 8 is not a multiple of 3


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 13, 16])
@pytest.mark.parametrize("n,kk,epilogue", [(8192, 8192, "relu"), (1000, 1024, "fast_gelu"), (64, 1024, ""),
                                           (4104, 2056, "add"), (72, 4096, "mul_add"), (520, 7176, "mul_add")])
def test_weight_streaming_rows(m, n, kk, epilogue):
    # M <= 4 with deep K runs on the weight-streaming CUDA-core kernel (benchmark configuration 5, M = 1), larger M
    # on the split-K tensor-core path; ragged N, K not a multiple of the unrolled step, residual epilogues
    k = _kernels()
    x = _rand((m, kk), 500, dist="uniform")
    w = _rand((n, kk), 501, scale=0.02)
    b = _rand((n,), 502, scale=0.1)
    nres = {"add": 1, "mul_add": 2}.get(epilogue, 0)
    d = [_rand((m, n), 503 + i) for i in range(nres)]
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue)
    assert k.device_status() == 0
    want = oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue)
    _close(y, want)
    y256 = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue, tile_n=256)
    _close(y256, want)                                # the tensor-core path on the same problem


def test_weight_streaming_rows_bf16_strided_and_permuted():
    k = _kernels()
    x = _rand((2, 2048), 510, dist="uniform", dtype=torch.bfloat16)
    w = _rand((512, 2048), 511, scale=0.02, dtype=torch.bfloat16)
    _close(k.gemm_rcr(x.cuda(), w.cuda(), None, alpha=0.5), oracle.gemm_rcr(x, w, None, alpha=0.5), atol=4e-2, rtol=4e-2)
    xh, wh, bh = x.half(), w.half(), _rand((512,), 512)
    buf = torch.full((2, 1024), 3.0, dtype=torch.float16, device="cuda")     # write into a column block of a wider row
    k.gemm_rcr(xh.cuda(), wh.cuda(), bh.cuda(), out=buf[:, 256:768])
    _close(buf[:, 256:768], oracle.gemm_rcr(xh, wh, bh))
    assert bool((buf[:, :256] == 3.0).all()) and bool((buf[:, 768:] == 3.0).all())
    y = k.gemm_rcr(xh.cuda(), wh.cuda(), bh.cuda(), permute_shape=(1, 2, 4))  # Permute5D store of the same rows
    _close(y, oracle.gemm_rcr_bias_permute(xh, wh, bh, (1, 2, 4)))


def test_reference_signature_entry_points():
    """The per-op entry points that take the reference's generated argument list."""
    import ctypes

    from aitemplate_b200 import _lib

    lib = _lib.load()
    m, n, kk = 200, 136, 64
    x = _rand((m, kk), 80)
    w = _rand((n, kk), 81, scale=0.1)
    b = _rand((n,), 82)
    d0 = _rand((m, n), 83)
    xg, wg, bg, dg = x.cuda(), w.cuda(), b.cuda(), d0.cuda()
    out = torch.empty((m, n), dtype=torch.float16, device="cuda")
    dims = [ctypes.c_int64(v) for v in (m, kk, n, kk, 0, 0)]
    refs = [ctypes.byref(v) for v in dims]
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.b200ait_gemm_rcr_bias_fast_gelu(xg.data_ptr(), wg.data_ptr(), bg.data_ptr(), out.data_ptr(), None, 1,
                                                  *refs, stream), "fast_gelu")
    assert (dims[4].value, dims[5].value) == (m, n)
    _close(out, oracle.gemm_rcr(x, w, b, epilogue="fast_gelu"))
    _lib.check(lib.b200ait_gemm_rcr_bias_add(xg.data_ptr(), wg.data_ptr(), bg.data_ptr(), dg.data_ptr(), out.data_ptr(),
                                            None, 1, *refs, stream), "add")
    _close(out, oracle.gemm_rcr(x, w, b, d0, epilogue="add"))
    # a null bias with a non-empty problem is rejected like the reference ("bias_ptr is null!")
    assert lib.b200ait_gemm_rcr_bias(xg.data_ptr(), wg.data_ptr(), None, out.data_ptr(), None, 1, *refs, stream) != 0
    assert "bias_ptr is null" in _lib.last_error()


def test_large_gemm_rows_sampled_against_oracle():
    # benchmark config 5 at M = 8192, N = K = 8192: the oracle checks 48 sampled rows (4 GFLOP on the host)
    k = _kernels()
    m, n, kk = 8192, 8192, 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.rand((m, kk), generator=g, device="cuda") * 2 - 1).half()
    w = (torch.randn((n, kk), generator=g, device="cuda") * 0.01).half()
    b = (torch.randn((n,), generator=g, device="cuda") * 0.01).half()
    y = k.gemm_rcr(x, w, b, epilogue="relu")
    rows = torch.randint(0, m, (48,), generator=torch.Generator().manual_seed(6))
    rows[0], rows[1] = 0, m - 1
    want = oracle.gemm_rcr(x[rows.cuda()], w, b, epilogue="relu")
    _close(y[rows.cuda()], want)
    # linearity in the residual: (x W^T + b + d) - (x W^T + b) == d up to two roundings
    d = (torch.randn((m, n), generator=g, device="cuda")).half()
    y0 = k.gemm_rcr(x, w, b, epilogue="")
    y1 = k.gemm_rcr(x, w, b, d, epilogue="add")
    assert float(((y1.float() - y0.float()) - d.float()).abs().max()) < 1e-2


@pytest.mark.parametrize(
    "m,n,kk,epilogue,split_k",
    [
        (128, 768, 3072, "add", 0),       # few tiles, deep K: the library splits on its own
        (384, 768, 3072, "fast_gelu", 0),  # BERT-base FFN2 at batch 1: K is deep enough for a split to pay
        (100, 520, 1000, "add_relu", 5),  # ragged M / N / K with a capped split count
        (64, 64, 4096, "", 0),
        (7, 264, 2048, "mul", 3),
        (128, 256, 512, "relu", 1),       # split-K switched off
    ],
)
def test_split_k_matches_oracle(m, n, kk, epilogue, split_k):
    k = _kernels()
    x = _rand((m, kk), 90, "uniform")
    w = _rand((n, kk), 91, scale=0.05)
    b = _rand((n,), 92, scale=0.1)
    d0 = _rand((m, n), 93)
    _, b1, _, _ = oracle.EPILOGUES[epilogue]
    if split_k != 1:
        assert k.gemm_workspace_bytes(1, m, n, kk, 0, split_k) > 0, "this shape is expected to split"
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), d0.cuda() if b1 else None, epilogue=epilogue, split_k=split_k)
    _close(y, oracle.gemm_rcr(x, w, b, d0 if b1 else None, epilogue=epilogue))


def test_short_k_is_not_split_by_the_library():
    """A split costs a second launch and a round trip of partial sums: below K = 2048 the library leaves K whole
    (BERT-base at batch 1: 384 x 768 x 768 runs in 8 us unsplit against 14 us in six splits)."""
    k = _kernels()
    m, n, kk = 384, 768, 768
    assert k.gemm_workspace_bytes(1, m, n, kk, 0, 0) == 0
    x, w, b = _rand((m, kk), 90, "uniform"), _rand((n, kk), 91, scale=0.05), _rand((n,), 92, scale=0.1)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), epilogue="fast_gelu")
    _close(y, oracle.gemm_rcr(x, w, b, epilogue="fast_gelu"))


def test_split_k_with_permuted_store():
    k = _kernels()
    s, h, d, bsz = 16, 2, 64, 4
    hid = h * d
    x = _rand((bsz * s, 2048), 94, scale=0.5)
    w = _rand((3 * hid, 2048), 95, scale=0.05)
    b = _rand((3 * hid,), 96, scale=0.1)
    assert k.gemm_workspace_bytes(1, bsz * s, 3 * hid, 2048) > 0
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), permute_shape=(s, 3, h))
    _close(y, oracle.gemm_rcr_bias_permute(x, w, b, (s, 3, h)))


@pytest.mark.parametrize("m", [5, 16, 17, 32, 33, 64, 100, 128, 129, 200, 256])
@pytest.mark.parametrize("n,kk,epilogue,dtype", [(8192, 8192, "relu", torch.float16), (4104, 2056, "add", torch.float16),
                                                   (2048, 4096, "mul_add", torch.float16),
                                                   (3000, 2304, "fast_gelu", torch.bfloat16),
                                                   (2052, 2048, "add_relu", torch.float16),
                                                   (16384, 2048, "tanh", torch.float16)])
def test_swapped_operand_weight_streaming(m, n, kk, epilogue, dtype):
    """5 <= M <= 128 against a big weight matrix runs with the operands swapped (weight rows on the MMA rows, the
    rows of X as the MMA's N = 16 to 128), K halved across a cluster of two CTAs whose partial sums meet in shared
    memory: ragged N (a partial last slab), K tails, every MMA width, residual epilogues, bf16, a row pitch that
    rules out 16-byte stores, and more slabs than clusters (the hand-shake that recycles the partial-sum buffer)."""
    k = _kernels()
    x = _rand((m, kk), 600, dist="uniform", dtype=dtype)
    w = _rand((n, kk), 601, scale=0.02, dtype=dtype)
    b = _rand((n,), 602, scale=0.1, dtype=dtype)
    nres = {"add": 1, "mul_add": 2, "add_relu": 1}.get(epilogue, 0)
    d = [_rand((m, n), 603 + i, dtype=dtype) for i in range(nres)]
    want = oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue)
    tol = 1e-2 if dtype == torch.float16 else 4e-2
    for _ in range(2):  # twice: the second call reuses the cluster-shared buffers of nothing (fresh launch), same result
        y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue)
        assert k.device_status() == 0
        _close(y, want, atol=tol, rtol=tol)
    # the tensor-core tile path on the same problem agrees
    y256 = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue, tile_n=256)
    _close(y256, want, atol=tol, rtol=tol)


@pytest.mark.parametrize("m,n,kk,epilogue", [(128, 320, 1280, "add"), (64, 128, 2048, "relu"), (100, 200, 768, "fast_gelu"),
                                              (16, 768, 320, ""), (32, 136, 264, "tanh"), (5, 128, 512, "mul"),
                                              (48, 1024, 576, "relu"), (128, 4096, 384 + 8, "")])
def test_swapped_operand_narrow_and_shallow_weights(m, n, kk, epilogue):
    """The edges of what the weight-streaming kernel takes: one or two slabs (N = 128 .. 320, a ragged single slab),
    and K down to 256 for M <= 32 (four to five k-blocks shared by a cluster of four); k-block counts that do not
    divide by the cluster size (5, 7, 9) must still give every rank a share."""
    k = _kernels()
    x = _rand((m, kk), 630, dist="uniform")
    w = _rand((n, kk), 631, scale=0.05)
    b = _rand((n,), 632, scale=0.1)
    nres = {"add": 1, "mul": 1}.get(epilogue, 0)
    d = [_rand((m, n), 633 + i) for i in range(nres)]
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue)
    assert k.device_status() == 0
    _close(y, oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue))
    y256 = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue, tile_n=128)
    _close(y256, oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue))


@pytest.mark.parametrize("m", [129, 145, 200])
@pytest.mark.parametrize("n,kk", [(16384, 2048), (20000, 2304), (1024, 4096)])
def test_swapped_operand_second_pass_with_idle_ranks(m, n, kk):
    """More than 128 rows of X go through the exchange in two passes; with M just above 128 some ranks have rows in
    the first pass only, and with more slabs than clusters they come round again: their exchange barrier must keep
    its own phase count."""
    k = _kernels()
    x = _rand((m, kk), 640, dist="uniform")
    w = _rand((n, kk), 641, scale=0.03)
    b = _rand((n,), 642, scale=0.1)
    want = oracle.gemm_rcr(x, w, b, epilogue="relu")
    for _ in range(10):
        y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), epilogue="relu")
        assert k.device_status() == 0
        _close(y, want, atol=1.5e-2, rtol=1.5e-2)


@pytest.mark.parametrize("m,n,kk", [(257, 768, 3072), (300, 1024, 2048), (512, 768, 3072), (700, 520, 2056),
                                    (1000, 1000, 2304), (1024, 1024, 4096), (2048, 256, 4096), (1900, 250, 4104),
                                    (1024, 128, 2048), (400, 8192, 2048), (513, 4100, 8192)])
@pytest.mark.parametrize("epilogue", ["relu", "add", "mul_add"])
def test_swapped_operand_row_groups(m, n, kk, epilogue):
    """More rows of X than one tile holds, against few weight slabs: the weight-streaming kernel takes X in groups
    of 32 to 256 rows (a ragged last group, a last group with a single row, ragged slabs, small and large weights)."""
    k = _kernels()
    x = _rand((m, kk), 650, dist="uniform")
    w = _rand((n, kk), 651, scale=0.03)
    b = _rand((n,), 652, scale=0.1)
    nres = {"add": 1, "mul_add": 2}.get(epilogue, 0)
    d = [_rand((m, n), 653 + i) for i in range(nres)]
    from aitemplate_b200 import _lib

    xd, wd, bd, dd = x.cuda(), w.cuda(), b.cuda(), [t.cuda() for t in d]
    launches = _lib.kernel_launch_count()
    y = k.gemm_rcr(xd, wd, bd, *dd, epilogue=epilogue)
    assert k.device_status() == 0
    if epilogue == "relu" or -(-m // 128) * -(-n // 128) <= 32:  # what the weight-streaming planner takes
        assert _lib.kernel_launch_count() - launches == 1  # one kernel: no split-K reduction pass
    _close(y, oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue), atol=1.5e-2, rtol=1.5e-2)


def test_swapped_operand_row_groups_permuted_store():
    """The grouped rows land where a fused output permutation sends them (row index = group base + row in group)."""
    k = _kernels()
    m, seq, h, hid = 768, 384, 4, 256  # [B * S, 3 * H * D] -> [3, B, H, S, D]
    x = _rand((m, 2048), 660, scale=0.5)
    w = _rand((3 * hid, 2048), 661, scale=0.05)
    b = _rand((3 * hid,), 662, scale=0.1)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), permute_shape=(seq, 3, h))
    assert k.device_status() == 0
    _close(y, oracle.gemm_rcr_bias_permute(x, w, b, (seq, 3, h)))


def test_swapped_operand_random_shapes():
    """Seeded random problems all over what the weight-streaming kernel takes (5 <= M <= 128, N >= 128, K >= 512, or
    K >= 256 with M <= 32): ragged slabs, k-block counts of every residue, every X-tile width, both cluster sizes."""
    import random

    k = _kernels()
    rng = random.Random(20240611)
    epilogues = ["", "relu", "fast_gelu", "add", "mul_add", "add_relu", "sigmoid"]
    for case in range(64):
        m = rng.choice([5, 8, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 127, 128, 129, 160, 192, 193, 255, 256])
        n = rng.choice([128, 136, 200, 256, 320, 333, 512, 1000, 1001, 2048, 3000, 4736, 4744, 6000, 9601])
        kk = 8 * rng.randint(32 if m <= 32 else 64, 400)
        epilogue = rng.choice(epilogues)
        x = _rand((m, kk), 700 + case, dist="uniform")
        w = _rand((n, kk), 800 + case, scale=0.03)
        b = _rand((n,), 900 + case, scale=0.1)
        nres = {"add": 1, "mul_add": 2, "add_relu": 1}.get(epilogue, 0)
        d = [_rand((m, n), 1000 + 2 * case + i) for i in range(nres)]
        y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue)
        assert k.device_status() == 0, (m, n, kk, epilogue)
        try:
            _close(y, oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue), atol=1.5e-2, rtol=1.5e-2)
        except AssertionError as e:
            raise AssertionError(f"m={m} n={n} k={kk} epilogue={epilogue!r}: {e}") from None


@pytest.mark.parametrize("m,n,kk", [(128, 8192, 2048), (96, 3072, 2048), (40, 1024, 4096), (256, 8192, 2048), (200, 2048, 2048)])
def test_swapped_operand_rows_do_not_depend_on_their_position(m, n, kk):
    """Which rank of the cluster finishes a row of X depends on the row's index; the K shares are added in rank
    order all the same, so X with its rows reversed gives Y with its rows reversed, bit for bit (clusters of two
    and of four)."""
    k = _kernels()
    x = _rand((m, kk), 620, dist="uniform").cuda()
    w = _rand((n, kk), 621, scale=0.02).cuda()
    b = _rand((n,), 622, scale=0.1).cuda()
    y = k.gemm_rcr(x, w, b, epilogue="relu")
    y_rev = k.gemm_rcr(x.flip(0).contiguous(), w, b, epilogue="relu")
    assert k.device_status() == 0
    assert torch.equal(y_rev.flip(0), y)


@pytest.mark.parametrize("m,seq", [(32, 16), (96, 32), (192, 64)])
def test_swapped_operand_permuted_store(m, seq):
    """The weight-streaming path writes the permuted [3, B, H, S, D] projection layout like the tile kernels do."""
    k = _kernels()
    h, hid = 16, 1024
    x = _rand((m, 2048), 610, scale=0.5)
    w = _rand((3 * hid, 2048), 611, scale=0.05)
    b = _rand((3 * hid,), 612, scale=0.1)
    y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), permute_shape=(seq, 3, h))
    assert k.device_status() == 0
    _close(y, oracle.gemm_rcr_bias_permute(x, w, b, (seq, 3, h)))


def test_tile_kernels_random_shapes():
    """Seeded random problems for the tile kernels (M > 128, or a tile hint): ragged M / N / K, every tile width
    including the CTA pairs, library-chosen and capped split-K, all epilogue families, both dtypes."""
    import random

    k = _kernels()
    rng = random.Random(20240613)
    epilogues = ["", "relu", "gelu", "fast_gelu", "add", "add_relu", "mul", "mul_add", "sigmoid_mul", "tanh", "add_add"]
    for case in range(40):
        m = rng.choice([129, 200, 256, 300, 511, 640, 1000, 1536])
        n = 8 * rng.randint(8, 160)
        kk = 8 * rng.randint(8, 300)
        epilogue = rng.choice(epilogues)
        dtype = torch.bfloat16 if rng.random() < 0.25 else torch.float16
        tile_n = rng.choice([0, 0, 0, 64, 128, 256, 512])
        split_k = rng.choice([0, 0, 1, 3]) if tile_n != 512 else 0
        x = _rand((m, kk), 5000 + case, dist="uniform", dtype=dtype)
        w = _rand((n, kk), 6000 + case, scale=0.03, dtype=dtype)
        b = _rand((n,), 7000 + case, scale=0.1, dtype=dtype)
        nres = {"add": 1, "add_relu": 1, "mul": 1, "mul_add": 2, "sigmoid_mul": 1, "add_add": 2}.get(epilogue, 0)
        d = [_rand((m, n), 8000 + 2 * case + i, dtype=dtype) for i in range(nres)]
        tol = 1.5e-2 if dtype == torch.float16 else 5e-2
        try:
            y = k.gemm_rcr(x.cuda(), w.cuda(), b.cuda(), *[t.cuda() for t in d], epilogue=epilogue, tile_n=tile_n,
                           split_k=split_k)
            assert k.device_status() == 0
            _close(y, oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue), atol=tol, rtol=tol)
        except AssertionError as e:
            raise AssertionError(f"m={m} n={n} k={kk} epilogue={epilogue!r} {dtype} tile_n={tile_n} split_k={split_k}: {e}") from None


def test_planned_weight_streaming_random_shapes():
    """Seeded random problems where the library's planner chooses among the weight-streaming kernels (weights of at
    most 16 MB, up to 64 output tiles): every group width and cluster size it can pick, ragged groups and slabs,
    k-block counts of every residue, every epilogue family (short store loop, activation pre-pass, long store loop),
    both dtypes. Each result must also be what the tile kernels give for the same problem, within rounding."""
    import random

    k = _kernels()
    rng = random.Random(20240701)
    epilogues = ["", "relu", "gelu", "fast_gelu", "tanh", "sigmoid", "add", "add_relu", "mul", "mul_add", "add_add", "sigmoid_mul"]
    for case in range(48):
        m = rng.choice([33, 64, 100, 129, 200, 256, 257, 384, 500, 512, 700, 1000, 1024])
        n = 8 * rng.randint(16, max(16, min(160, 8192 // max(m, 128) * 16)))
        kk = 8 * rng.randint(32, 520)
        epilogue = rng.choice(epilogues)
        dtype = torch.bfloat16 if rng.random() < 0.25 else torch.float16
        x = _rand((m, kk), 21000 + case, dist="uniform", dtype=dtype)
        w = _rand((n, kk), 22000 + case, scale=0.03, dtype=dtype)
        b = _rand((n,), 23000 + case, scale=0.1, dtype=dtype)
        nres = {"add": 1, "add_relu": 1, "mul": 1, "mul_add": 2, "sigmoid_mul": 1, "add_add": 2}.get(epilogue, 0)
        d = [_rand((m, n), 24000 + 2 * case + i, dtype=dtype) for i in range(nres)]
        tol = 1.5e-2 if dtype == torch.float16 else 5e-2
        dev = [t.cuda() for t in (x, w, b, *d)]
        try:
            y = k.gemm_rcr(*dev, epilogue=epilogue)
            assert k.device_status() == 0
            _close(y, oracle.gemm_rcr(x, w, b, *d, epilogue=epilogue), atol=tol, rtol=tol)
            y_tile = k.gemm_rcr(*dev, epilogue=epilogue, tile_n=128, split_k=1)
            _close(y, y_tile.float().cpu(), atol=tol, rtol=tol)
        except AssertionError as e:
            raise AssertionError(f"m={m} n={n} k={kk} epilogue={epilogue!r} {dtype}: {e}") from None


def test_batched_and_row_major_random_shapes():
    """Seeded random problems for bmm_rcr, bmm_rrr (B stored [K, N]), gemm_rrr and a broadcast operand."""
    import random

    k = _kernels()
    rng = random.Random(20240616)
    for case in range(30):
        bsz = rng.choice([1, 2, 5, 16])
        m = rng.choice([1, 8, 100, 128, 200, 384])
        n = 8 * rng.randint(1, 60)
        kk = 8 * rng.randint(1, 80)
        alpha = rng.choice([1.0, 0.125])
        a = _rand((bsz, m, kk), 12000 + case, dist="uniform")
        try:
            if case % 3 == 0:
                b = _rand((bsz, n, kk), 13000 + case, scale=0.1)
                _close(k.bmm_rcr(a.cuda(), b.cuda(), alpha=alpha), oracle.bmm_rcr(a, b, alpha=alpha), atol=1.5e-2, rtol=1.5e-2)
                b1 = b[:1]  # one B for every batch
                _close(k.bmm_rcr(a.cuda(), b1.cuda(), alpha=alpha), oracle.bmm_rcr(a, b1.expand(bsz, n, kk), alpha=alpha),
                       atol=1.5e-2, rtol=1.5e-2)
            elif case % 3 == 1:
                b = _rand((bsz, kk, n), 13000 + case, scale=0.1)
                _close(k.bmm_rrr(a.cuda(), b.cuda(), alpha=alpha), oracle.bmm_rrr(a, b, alpha=alpha), atol=1.5e-2, rtol=1.5e-2)
            else:
                w = _rand((kk, n), 13000 + case, scale=0.1)
                bias = _rand((n,), 14000 + case, scale=0.1)
                _close(k.gemm_rrr(a[0].cuda(), w.cuda(), bias.cuda()), oracle.gemm_rrr(a[0], w, bias), atol=1.5e-2, rtol=1.5e-2)
        except AssertionError as e:
            raise AssertionError(f"case {case}: batch={bsz} m={m} n={n} k={kk} alpha={alpha}: {e}") from None

