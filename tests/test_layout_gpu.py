"""Bit-exact GPU checks of concatenate / split / permute and parity of the element-wise chain.

The reference compares these ops with torch.equal (tests/unittest/ops/test_concatenate.py:74,132,204,
test_split.py:107,171, test_permute.py); so do these tests. Includes the benchmark case: four
[8192, 1024] fp16 tensors concatenated on dim 1 and split back.
"""
import pytest
import torch

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu


def _rand(shape, seed, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    if dtype in (torch.int32, torch.int64, torch.uint8):
        return torch.randint(0, 100, shape, generator=g).to(dtype)
    return torch.randn(shape, generator=g).to(dtype)


@pytest.mark.parametrize(
    "shapes,dim",
    [
        ([(8192, 1024)] * 4, 1),
        ([(2, 3, 4), (2, 5, 4), (2, 1, 4)], 1),
        ([(3, 7), (5, 7)], 0),
        ([(4, 3), (4, 5), (4, 9)], -1),
        ([(2, 2, 3, 1), (2, 2, 3, 7)], 3),
        ([(1024, 0), (1024, 8)], 1),
        ([(5,), (9,), (1,)], 0),
    ],
)
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.int64])
def test_concatenate_and_split_round_trip(shapes, dim, dtype):
    from aitemplate_b200 import kernels

    if dtype != torch.float16 and shapes[0] == (8192, 1024):
        pytest.skip("full-size case runs in fp16 only")
    xs = [_rand(s, i, dtype) for i, s in enumerate(shapes)]
    y = kernels.concatenate([x.cuda() for x in xs], dim)
    want = oracle.concatenate(xs, dim)
    assert torch.equal(y.cpu(), want)
    sizes = [s[dim] for s in shapes]
    parts = kernels.split(y, sizes, dim)
    for p, x in zip(parts, xs):
        assert torch.equal(p.cpu(), x)


def test_concatenate_masked_inputs_are_left_untouched():
    from aitemplate_b200 import kernels

    a, b, c = _rand((16, 8), 1), _rand((16, 24), 2), _rand((16, 8), 3)
    out = torch.full((16, 40), 7.0, dtype=torch.float16, device="cuda")
    kernels.concatenate([a.cuda(), b.cuda(), c.cuda()], 1, input_masks=[True, False, True], out=out)
    got = out.cpu()
    assert torch.equal(got[:, :8], a) and torch.equal(got[:, 32:], c)
    assert bool((got[:, 8:32] == 7.0).all())


@pytest.mark.parametrize("size,dim,shape", [(2, 0, (5, 6)), (4, 1, (3, 10, 2)), (1, 0, (3, 64, 12, 16))])
def test_split_by_chunk_size_with_ragged_tail(size, dim, shape):
    from aitemplate_b200 import kernels

    x = _rand(shape, 4)
    got = kernels.split(x.cuda(), size, dim)
    want = oracle.split(x, size, dim)
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert torch.equal(g.cpu(), w)


@pytest.mark.parametrize(
    "shape,dims",
    [
        ((2, 4096, 8, 40), (0, 2, 1, 3)),  # UNet q/k/v head split
        ((3, 5, 7), (0, 2, 1)),
        ((3, 5, 7), (1, 0, 2)),
        ((3, 5, 7), (2, 1, 0)),
        ((64, 100), (1, 0)),
        ((200, 66), (1, 0)),               # 16-bit: 64 x 64 tiles with 32-bit accesses, ragged in both directions
        ((3, 130, 258), (0, 2, 1)),
        ((5, 64, 384), (0, 2, 1)),
        ((2, 65, 128), (0, 2, 1)),         # odd R: the 32 x 32 kernel
        ((2, 3, 4, 5, 6), (4, 0, 3, 1, 2)),
        ((7, 1, 9), (2, 1, 0)),
        ((4, 6), (0, 1)),
        ((2, 384, 3, 12, 64), (2, 0, 3, 1, 4)),
    ],
)
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_permute(shape, dims, dtype):
    from aitemplate_b200 import kernels

    x = _rand(shape, 5, dtype)
    assert torch.equal(kernels.permute(x.cuda(), dims).cpu(), oracle.permute(x, dims))


@pytest.mark.parametrize(
    "shapes,steps",
    [
        ([(2, 4096, 320), (2, 4096, 320)], [("add", 1)]),
        ([(128, 768), (768,)], [("add", 1), ("fast_gelu", None)]),
        ([(33, 7), (33, 1)], [("mul", 1), ("relu", None)]),
        ([(16, 64)], [("gelu", None)]),
        ([(16, 64)], [("mul", 0.5), ("add", 1.0), ("tanh", None)]),
        ([(4, 1, 8), (1, 5, 8), (8,)], [("add", 1), ("mul", 2), ("sigmoid", None)]),
        ([(1,), (9, 16)], [("sub", 1)]),
    ],
)
def test_elementwise_chain(shapes, steps):
    from aitemplate_b200 import kernels

    xs = [_rand(s, 10 + i) for i, s in enumerate(shapes)]
    y = kernels.elementwise([x.cuda() for x in xs], steps)
    want = oracle.elementwise(xs, steps)
    got = y.float().cpu()
    assert got.shape == want.shape
    assert bool(((got - want).abs() <= 1e-2 + 1e-2 * want.abs()).all())


def test_random_shapes_bit_exact():
    """Seeded random concatenate / split / permute problems (ranks 2-5, odd extents, every dim, both 16-bit types and
    fp32): results must equal torch's bit for bit."""
    import itertools
    import random

    from aitemplate_b200 import kernels

    rng = random.Random(20240615)
    for case in range(40):
        rank = rng.randint(2, 5)
        dtype = rng.choice([torch.float16, torch.bfloat16, torch.float32])
        shape = [rng.choice([1, 2, 3, 5, 8, 17, 32, 63]) for _ in range(rank)]
        dim = rng.randrange(rank)
        gen = torch.Generator().manual_seed(11000 + case)
        xs = []
        for i in range(rng.randint(1, 4)):
            s = list(shape)
            s[dim] = rng.choice([1, 2, 7, 16, 40])
            xs.append(torch.randn(s, generator=gen).to(dtype))
        want = torch.cat(xs, dim)
        got = kernels.concatenate([x.cuda() for x in xs], dim)
        assert torch.equal(got.cpu(), want), f"concatenate {[tuple(x.shape) for x in xs]} dim {dim} {dtype}"
        parts = kernels.split(got, [x.shape[dim] for x in xs], dim)
        for p, x in zip(parts, xs):
            assert torch.equal(p.cpu(), x), f"split {tuple(want.shape)} dim {dim} {dtype}"
        dims = list(range(rank))
        rng.shuffle(dims)
        x = torch.randn(shape, generator=gen).to(dtype)
        assert torch.equal(kernels.permute(x.cuda(), dims).cpu(), x.permute(dims).contiguous()), f"permute {shape} {dims} {dtype}"
