"""GPU parity of layernorm and softmax against the CPU oracle, through the C ABI.

Shapes follow tests/unittest/ops/test_layernorm.py:35-205 (batch 50/900/1024, N=1496, gamma/beta None,
eps 1e-5 and 0.1, multi-dim normalized shape) and test_softmax.py:72-225 (the K list, inner dims,
zero batch), plus the benchmark memory-bound sweep shapes. Tolerances are the reference's:
1e-3 for layernorm, 1e-2 for softmax.
"""
import pytest
import torch

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0, dist="normal", dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    t = torch.rand(shape, generator=g) if dist == "uniform" else torch.randn(shape, generator=g)
    return (t * scale).to(dtype)


def _close(got, want, tol):
    got = got.float().cpu()
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    err = (got - want).abs()
    assert bool((err <= tol + tol * want.abs()).all()), f"max abs err {float(err.max()):.4g}"


@pytest.mark.parametrize("m", [50, 900, 1024])
@pytest.mark.parametrize("n", [1496, 768, 1024, 4096, 320, 8, 1001, 5000, 8192])
def test_layernorm(m, n):
    from aitemplate_b200 import kernels

    x = _rand((m, n), 1)
    g = (_rand((n,), 2, dist="uniform") + 0.5).half()
    b = _rand((n,), 3, scale=0.1)
    y = kernels.layernorm(x.cuda(), g.cuda(), b.cuda(), eps=1e-5)
    _close(y, oracle.layernorm(x, g, b, 1e-5), 1e-3 * 2)


@pytest.mark.parametrize("use_gamma,use_beta", [(False, False), (True, False), (False, True)])
@pytest.mark.parametrize("eps", [1e-5, 0.1, 1e-12])
def test_layernorm_optional_affine(use_gamma, use_beta, eps):
    from aitemplate_b200 import kernels

    x = _rand((123, 1496), 4, scale=3.0)
    g = _rand((1496,), 5) if use_gamma else None
    b = _rand((1496,), 6) if use_beta else None
    y = kernels.layernorm(x.cuda(), g.cuda() if use_gamma else None, b.cuda() if use_beta else None, eps=eps)
    _close(y, oracle.layernorm(x, g, b, eps), 2e-3)


def test_layernorm_multi_dim_normalized_shape_and_zero_rows():
    from aitemplate_b200 import kernels

    x = _rand((7, 5, 16, 24), 7)
    g = _rand((16, 24), 8)
    b = _rand((16, 24), 9)
    y = kernels.layernorm(x.cuda(), g.cuda(), b.cuda(), normalized_ndim=2)
    _close(y, oracle.layernorm(x, g, b, normalized_ndim=2), 2e-3)
    z = torch.zeros((0, 64), dtype=torch.float16, device="cuda")
    assert tuple(kernels.layernorm(z, None, None).shape) == (0, 64)


def test_layernorm_bf16():
    from aitemplate_b200 import kernels

    x = _rand((64, 768), 10, dtype=torch.bfloat16)
    g = _rand((768,), 11, dtype=torch.bfloat16)
    b = _rand((768,), 12, dtype=torch.bfloat16)
    y = kernels.layernorm(x.cuda(), g.cuda(), b.cuda())
    _close(y, oracle.layernorm(x, g, b), 2e-2)


@pytest.mark.parametrize("k", [6, 11, 33, 1409, 18, 66, 1154, 124, 132, 1924, 72, 264, 3848, 12500, 1024, 4096])
def test_softmax_last_dim(k):
    from aitemplate_b200 import kernels

    x = _rand((37, k), 20, scale=2.0)
    _close(kernels.softmax(x.cuda(), -1), oracle.softmax(x, -1), 1e-2)
    s = kernels.softmax(x.cuda(), -1).float().sum(-1)
    assert float((s - 1).abs().max()) < 2e-2


@pytest.mark.parametrize("shape,dim", [((4, 33, 5), 1), ((3, 7, 2, 4), 1), ((2, 1024, 8), 1), ((6, 5), 0),
                                       ((2, 3, 1024), 2)])
def test_softmax_inner_dims(shape, dim):
    from aitemplate_b200 import kernels

    x = _rand(shape, 21, scale=2.0)
    _close(kernels.softmax(x.cuda(), dim), oracle.softmax(x, dim), 1e-2)


def test_softmax_extremes_and_zero_batch():
    from aitemplate_b200 import kernels

    x = torch.full((4, 1024), -60000.0, dtype=torch.float16)
    x[:, 5] = 60000.0
    y = kernels.softmax(x.cuda(), -1).float().cpu()
    assert torch.equal(y.argmax(-1), torch.full((4,), 5))
    assert float((y[:, 5] - 1).abs().max()) < 1e-3
    z = torch.zeros((0, 64), dtype=torch.float16, device="cuda")
    assert tuple(kernels.softmax(z, -1).shape) == (0, 64)


def test_full_size_rows_are_independent_and_normalised():
    """benchmark memory-bound sweep at full size: layernorm [65536, 1024] and softmax [64, 1024, 1024]
    (one eighth of the batch) checked through size-independent properties plus sampled rows."""
    from aitemplate_b200 import kernels

    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((65536, 1024), generator=g, device="cuda").half()
    gamma = (torch.rand((1024,), generator=g, device="cuda") + 0.5).half()
    beta = (torch.randn((1024,), generator=g, device="cuda") * 0.1).half()
    y = kernels.layernorm(x, gamma, beta, eps=1e-5)
    rows = torch.tensor([0, 1, 31, 32, 4095, 65535, 12345, 40000])
    _close(y[rows.cuda()], oracle.layernorm(x[rows.cuda()], gamma, beta, 1e-5), 2e-3)
    # with gamma = 1, beta = 0 every row has mean 0 and variance 1
    yn = kernels.layernorm(x, None, None, eps=1e-5).float()
    assert float(yn.mean(-1).abs().max()) < 2e-3
    assert float((yn.var(-1, unbiased=False) - 1).abs().max()) < 5e-3
    s = torch.randn((64, 1024, 1024), generator=g, device="cuda").mul_(2).half()
    p = kernels.softmax(s, -1)
    assert float((p.float().sum(-1) - 1).abs().max()) < 2e-2
    _close(p[3, 100:108], oracle.softmax(s[3, 100:108], -1), 1e-2)


def test_random_shapes():
    """Seeded random row counts and row lengths (odd lengths, lengths around the vector widths and the per-warp and
    per-block limits of the kernels) for layernorm and for softmax over the last and over an inner dimension."""
    import random

    from aitemplate_b200 import kernels

    rng = random.Random(20240614)
    for case in range(40):
        m = rng.choice([1, 3, 31, 64, 257, 1000])
        n = rng.choice([1, 2, 7, 8, 9, 63, 64, 65, 255, 256, 320, 511, 777, 1024, 1025, 2048, 3000, 4097, 9000, 16384])
        x = _rand((m, n), 9000 + case, scale=rng.choice([0.1, 1.0, 8.0]))
        g, b = (_rand((n,), 9100 + case, dist="uniform") + 0.5).half(), _rand((n,), 9200 + case, scale=0.1)
        try:
            _close(kernels.layernorm(x.cuda(), g.cuda(), b.cuda(), eps=1e-5), oracle.layernorm(x, g, b, 1e-5), 4e-3)
            _close(kernels.softmax(x.cuda(), -1), oracle.softmax(x, -1), 1e-2)
            inner = rng.choice([2, 5, 16])
            x3 = _rand((rng.choice([1, 4]), max(1, min(n, 300)), inner), 9300 + case)
            _close(kernels.softmax(x3.cuda(), 1), oracle.softmax(x3, 1), 1e-2)
        except AssertionError as e:
            raise AssertionError(f"m={m} n={n}: {e}") from None


@pytest.mark.parametrize("n", [1030, 1031, 4100, 5001, 33000, 40000, 65537, 102400, 102401, 120000])
def test_rows_staged_in_shared_memory(n):
    """Row lengths the vector kernels do not take (not a multiple of 8 elements, or above 32768): up to 100 K elements
    the row is staged in shared memory (even lengths two elements at a time), above that it is read three times."""
    from aitemplate_b200 import kernels

    m = 9
    x = _rand((m, n), 31, scale=2.0)
    g, b = (_rand((n,), 32, dist="uniform") + 0.5).half(), _rand((n,), 33, scale=0.1)
    _close(kernels.layernorm(x.cuda(), g.cuda(), b.cuda(), eps=1e-5), oracle.layernorm(x, g, b, 1e-5), 4e-3)
    _close(kernels.layernorm(x.cuda(), None, None, eps=1e-5), oracle.layernorm(x, None, None, 1e-5), 4e-3)
    _close(kernels.softmax(x.cuda(), -1), oracle.softmax(x, -1), 1e-2)
    xb = x.to(torch.bfloat16)
    _close(kernels.softmax(xb.cuda(), -1), oracle.softmax(xb, -1), 2e-2)
    # a view that starts at an odd element: 2-byte aligned rows only
    flat = torch.zeros(m * n + 1, dtype=torch.float16)
    flat[1:] = x.reshape(-1)
    odd = flat.cuda()[1:].view(m, n)
    _close(kernels.softmax(odd, -1), oracle.softmax(x, -1), 1e-2)
