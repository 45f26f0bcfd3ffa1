"""GPU parity of mem_eff_attention against the CPU oracle, through the C ABI.

Shapes follow tests/unittest/ops/test_attention.py:456-742 ((B16,H4,S8,d=20) and (B16,H16,S1024,d=64)
scaled to what the host oracle finishes in seconds), :847-1010 (cross attention, Sq != Skv), and the
benchmark configurations (BERT S=384 D=64; UNet D=40 with Skv=4096 and Skv=77).
The reference's tolerance is 1e-3 against an fp16 torch result; against the fp32 oracle the bound
is atol = rtol = 1e-2 with a tighter 4e-3 absolute check on top. Padded variable lengths (lengths_kv / lengths_q)
follow test_attention.py:456-742 with variable_seq_length_kv / variable_seq_length_q.
"""
import pytest
import torch

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def _check(q, k, v, causal=False, atol=1e-2, tight=4e-3):
    from aitemplate_b200 import kernels

    out = kernels.mem_eff_attention(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    want = oracle.mem_eff_attention(q, k, v, causal=causal)
    got = out.float().cpu()
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    err = (got - want).abs()
    assert bool((err <= atol + 1e-2 * want.abs()).all()), f"max abs err {float(err.max()):.4g}"
    assert float(err.max()) < tight, f"max abs err {float(err.max()):.4g}"


@pytest.mark.parametrize(
    "b,h,sq,skv,d",
    [
        (16, 4, 8, 8, 20),      # CUDA-core kernel (head dim not a multiple of 8)
        (2, 12, 384, 384, 64),  # BERT-base
        (2, 4, 1024, 1024, 64),
        (1, 2, 4096, 4096, 40),  # UNet self-attention
        (2, 8, 4096, 77, 40),    # UNet cross-attention
        (3, 2, 200, 129, 64),    # ragged query and key tails
        (2, 2, 128, 128, 128),   # two 64-wide head-dim chunks
        (1, 3, 130, 260, 96),
        (2, 2, 64, 50, 8),
    ],
)
def test_non_causal(b, h, sq, skv, d):
    q = _rand((b, h, sq, d), 1)
    k = _rand((b, h, skv, d), 2)
    v = _rand((b, h, skv, d), 3)
    _check(q, k, v)


@pytest.mark.parametrize("b,h,s,d", [(2, 4, 384, 64), (1, 2, 300, 40), (4, 2, 8, 20)])
def test_causal(b, h, s, d):
    q = _rand((b, h, s, d), 4)
    k = _rand((b, h, s, d), 5)
    v = _rand((b, h, s, d), 6)
    _check(q, k, v, causal=True)


def test_large_scores_stay_finite():
    # rows whose maximum moves between key blocks exercise the running-max rescale
    q = _rand((1, 2, 256, 64), 7, scale=4.0)
    k = _rand((1, 2, 512, 64), 8, scale=4.0)
    v = _rand((1, 2, 512, 64), 9)
    _check(q, k, v, tight=8e-3)


def test_different_value_head_size():
    q = _rand((2, 2, 256, 64), 10)
    k = _rand((2, 2, 192, 64), 11)
    v = _rand((2, 2, 192, 32), 12)
    _check(q, k, v)


def test_bf16():
    q = _rand((2, 2, 256, 64), 13, dtype=torch.bfloat16)
    k = _rand((2, 2, 256, 64), 14, dtype=torch.bfloat16)
    v = _rand((2, 2, 256, 64), 15, dtype=torch.bfloat16)
    _check(q, k, v, atol=3e-2, tight=3e-2)


def test_zero_batch():
    from aitemplate_b200 import kernels

    z = torch.zeros((0, 4, 16, 64), dtype=torch.float16, device="cuda")
    assert tuple(kernels.mem_eff_attention(z, z, z).shape) == (0, 16, 4, 64)


# ---- packed variable-length attention (ops.flash_attention): tests/unittest/ops/test_attention.py:200-330 builds
# qkv [total, 3, H, D] + cu_seqlens and compares with attention_ref per sequence
@pytest.mark.parametrize("lengths,h,d,causal", [
    ([384] * 4, 12, 64, False),            # the BERT case: equal lengths
    ([384, 100, 1, 257, 130], 4, 64, False),
    ([384, 100, 1, 257, 130], 4, 64, True),
    ([77, 300, 128], 3, 32, False),
    ([512, 129], 2, 128, False),
    ([64, 0, 200], 2, 16, False),           # an empty sequence in the middle
])
def test_flash_attention_packed_variable_length(lengths, h, d, causal):
    from aitemplate_b200 import kernels

    total = sum(lengths)
    qkv = _rand((total, 3, h, d), 21)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    out = kernels.flash_attention(qkv.cuda(), cu.cuda(), max(lengths), causal=causal)
    assert kernels.device_status() == 0
    assert tuple(out.shape) == (total, h, d)
    got = out.float().cpu()
    for b, n in enumerate(lengths):
        if n == 0:
            continue
        lo = int(cu[b])
        q, k, v = (qkv[lo:lo + n, i].permute(1, 0, 2).unsqueeze(0) for i in range(3))  # [1, H, n, D]
        want = oracle.mem_eff_attention(q, k, v, causal=causal)[0]  # [n, H, D]
        err = (got[lo:lo + n] - want).abs()
        assert bool((err <= 1e-2 + 1e-2 * want.abs()).all()) and float(err.max()) < 4e-3, (b, float(err.max()))


@pytest.mark.parametrize("b,h,sq,skv,d,causal", [(2, 8, 1024, 1024, 40, False), (2, 8, 512, 77, 40, False),
                                                  (3, 4, 200, 200, 64, True), (1, 2, 130, 260, 96, False)])
def test_strided_operands_read_in_place(b, h, sq, skv, d, causal):
    """q, k, v stored [B, S, H, D] (a projection output) and handed over as permuted views: no copy is made."""
    from aitemplate_b200 import kernels

    qs, ks, vs = _rand((b, sq, h, d), 31), _rand((b, skv, h, d), 32), _rand((b, skv, h, d), 33)
    qd, kd, vd = qs.cuda(), ks.cuda(), vs.cuda()
    out = kernels.mem_eff_attention_strided(qd.permute(0, 2, 1, 3), kd.permute(0, 2, 1, 3), vd.permute(0, 2, 1, 3),
                                            causal=causal)
    assert kernels.device_status() == 0
    want = oracle.mem_eff_attention(qs.permute(0, 2, 1, 3), ks.permute(0, 2, 1, 3), vs.permute(0, 2, 1, 3), causal=causal)
    err = (out.float().cpu() - want).abs()
    assert bool((err <= 1e-2 + 1e-2 * want.abs()).all()) and float(err.max()) < 4e-3, float(err.max())
    # mixed: q in place, k and v contiguous [B, H, S, D]
    out2 = kernels.mem_eff_attention_strided(qd.permute(0, 2, 1, 3), kd.permute(0, 2, 1, 3).contiguous(),
                                             vd.permute(0, 2, 1, 3).contiguous(), causal=causal)
    assert torch.equal(out2, out)


def test_random_shapes():
    """Seeded random problems: every head size the tensor-core kernel takes (multiples of 8 up to 128), ragged query
    and key tails, one to a few dozen key blocks, causal or not, different value head sizes."""
    import random

    rng = random.Random(20240612)
    for case in range(32):
        b, h = rng.randint(1, 3), rng.randint(1, 5)
        d = rng.choice([8, 16, 24, 32, 40, 48, 64, 72, 80, 96, 128])
        causal = rng.random() < 0.35
        sq = rng.choice([1, 7, 64, 100, 128, 129, 200, 384, 500, 777])
        skv = sq if causal else rng.choice([1, 13, 63, 64, 65, 77, 128, 191, 320, 1000, 1500])
        dv = d if rng.random() < 0.7 else rng.choice([8, 32, 64, 128])
        q = _rand((b, h, sq, d), 2000 + case)
        k = _rand((b, h, skv, d), 3000 + case)
        v = _rand((b, h, skv, dv), 4000 + case)
        try:
            _check(q, k, v, causal=causal)
        except AssertionError as e:
            raise AssertionError(f"b={b} h={h} sq={sq} skv={skv} d={d} dv={dv} causal={causal}: {e}") from None


def test_flash_attention_random_lengths():
    """Seeded random packed batches: sequence lengths from 0 to a few hundred in any mix, several head sizes, causal or
    not; every sequence is checked against the oracle on its own rows."""
    import random

    from aitemplate_b200 import kernels

    rng = random.Random(20240617)
    for case in range(12):
        nseq = rng.randint(1, 7)
        lengths = [rng.choice([0, 1, 5, 63, 64, 65, 127, 128, 129, 200, 333, 400]) for _ in range(nseq)]
        if sum(lengths) == 0:
            lengths[0] = 17
        h, d, causal = rng.randint(1, 4), rng.choice([16, 32, 64, 128]), rng.random() < 0.4
        total = sum(lengths)
        qkv = _rand((total, 3, h, d), 15000 + case)
        cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
        out = kernels.flash_attention(qkv.cuda(), cu.cuda(), max(lengths), causal=causal)
        assert kernels.device_status() == 0
        got = out.float().cpu()
        for b, n in enumerate(lengths):
            if n == 0:
                continue
            lo = int(cu[b])
            q, k, v = (qkv[lo:lo + n, i].permute(1, 0, 2).unsqueeze(0) for i in range(3))
            want = oracle.mem_eff_attention(q, k, v, causal=causal)[0]
            err = (got[lo:lo + n] - want).abs()
            assert bool((err <= 1e-2 + 1e-2 * want.abs()).all()) and float(err.max()) < 4e-3, \
                f"lengths={lengths} h={h} d={d} causal={causal} sequence {b}: max abs err {float(err.max()):.4g}"


def _check_lengths(b, h, sq, skv, d, lengths_kv, lengths_q, causal=False, seed=50):
    from aitemplate_b200 import kernels

    q, k, v = _rand((b, h, sq, d), seed), _rand((b, h, skv, d), seed + 1), _rand((b, h, skv, d), seed + 2)
    lkv = None if lengths_kv is None else torch.tensor(lengths_kv, dtype=torch.int32)
    lq = None if lengths_q is None else torch.tensor(lengths_q, dtype=torch.int32)
    sentinel = 7.0
    out = torch.full((b, sq, h, d), sentinel, dtype=torch.float16, device="cuda")
    kernels.mem_eff_attention(q.cuda(), k.cuda(), v.cuda(), causal=causal, out=out,
                              lengths_kv=None if lkv is None else lkv.reshape(b, 1).cuda(),
                              lengths_q=None if lq is None else lq.cuda())
    assert kernels.device_status() == 0
    got = out.float().cpu()
    want = oracle.mem_eff_attention(q, k, v, causal=causal, lengths_kv=lkv, lengths_q=lq)
    for i in range(b):
        rows = sq if lq is None else min(int(lq[i]), sq)
        assert bool((got[i, rows:] == sentinel).all()), f"batch {i}: rows past lengths_q were written"
        g, w = got[i, :rows], want[i, :rows]
        if lkv is not None and int(lkv[i]) == 0:
            assert bool(torch.isnan(g).all()) and bool(torch.isnan(w).all()), f"batch {i}: no keys must give NaN"
            continue
        assert bool(torch.isfinite(g).all()), f"batch {i}"
        err = (g - w).abs()
        assert bool((err <= 1e-2 + 1e-2 * w.abs()).all()) and (rows == 0 or float(err.max()) < 4e-3), \
            f"batch {i}: max abs err {float(err.max()) if rows else 0:.4g}"


@pytest.mark.parametrize("d", [64, 40, 128, 20])  # 20: the CUDA-core kernel
@pytest.mark.parametrize("var_kv,var_q", [(True, False), (False, True), (True, True)])
def test_padded_variable_lengths(d, var_kv, var_q):
    b, h, s = 6, 3, 200
    lengths_kv = [200, 0, 1, 64, 65, 137] if var_kv else None
    lengths_q = [0, 200, 128, 129, 5, 77] if var_q else None
    _check_lengths(b, h, s, s, d, lengths_kv, lengths_q)


def test_padded_variable_lengths_causal_and_cross():
    _check_lengths(4, 2, 256, 256, 64, [256, 100, 0, 31], [256, 256, 10, 200], causal=True)
    _check_lengths(3, 4, 384, 128, 64, [128, 64, 7], None)           # Skv a multiple of the key block: masks still apply
    _check_lengths(2, 2, 64, 300, 32, [300, 150], [64, 1])
    _check_lengths(2, 2, 130, 70, 20, [70, 0], [130, 129], causal=False)


def test_padded_variable_lengths_random():
    import random

    rng = random.Random(20240702)
    for case in range(16):
        b, h = rng.randint(1, 5), rng.randint(1, 4)
        d = rng.choice([16, 32, 64, 80, 128, 20])
        sq, skv = rng.choice([1, 64, 129, 300, 512]), rng.choice([1, 63, 64, 200, 384])
        causal = rng.random() < 0.3
        if causal:
            skv = sq
        lkv = [rng.choice([0, 1, skv // 2, skv, skv + 5]) for _ in range(b)] if rng.random() < 0.8 else None
        lq = [rng.choice([0, 1, sq // 2, sq, sq + 3]) for _ in range(b)] if rng.random() < 0.6 else None
        try:
            _check_lengths(b, h, sq, skv, d, lkv, lq, causal=causal, seed=100 + 3 * case)
        except AssertionError as e:
            raise AssertionError(f"b={b} h={h} sq={sq} skv={skv} d={d} causal={causal} lkv={lkv} lq={lq}: {e}") from None
