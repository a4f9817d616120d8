"""Host checks of the tile layout and of the exact-arithmetic tricks behind the tensor-core GEMV."""

import pytest
import torch

from megakernels_b200 import _lib
from megakernels_b200.pack import as_bytes, pack_rows, plan_rows, unpack_rows


def test_plan_rows_mirror_matches_library(lib_built):
    for rows, unit in ((8224, 1), (7168, 2), (151936, 1), (1024, 1)):
        for cta in (0, 1, 73, 147):
            assert plan_rows(rows, unit, cta, 148) == _lib.plan_rows(rows, unit, cta, 148)


@pytest.mark.parametrize("n,rb,unit", [(8224, 1024, 1), (5120, 2048, 1), (1024, 2048, 1), (1024, 3584, 1),
                                       (1024, 7168, 1), (7168, 1024, 2), (1024, 4096, 1), (4099, 1024, 1)])
def test_pack_is_a_permutation_within_groups_and_invertible(n, rb, unit):
    g = torch.Generator().manual_seed(n + rb)
    w = torch.randint(0, 256, (n, rb), dtype=torch.uint8, generator=g)
    p = pack_rows(w, unit, 148, 32768)
    assert p.shape == w.shape and not torch.equal(p, w)
    assert torch.equal(unpack_rows(p, unit, 148, 32768), w)
    # a CTA's slice holds exactly its own rows' bytes
    r0, r1 = plan_rows(n, unit, 5, 148)
    assert torch.equal(p[r0:r1].flatten().sort().values, w[r0:r1].flatten().sort().values)


def test_tile_addressing_as_the_kernel_reads_it():
    """Lane (g, t) of a warp reads 16 bytes at group_base + (kb * rows_in_group + g) * 64 + t * 16 and
    must find bytes [64 kb + 16 t, +16) of row g."""
    n, rb = 1024, 2048
    w = torch.arange(n * rb, dtype=torch.int64).remainder(251).to(torch.uint8).view(n, rb)
    p = pack_rows(w, 1, 148, 32768).flatten()
    r0, r1 = plan_rows(n, 1, 9, 148)
    ng = r1 - r0                                  # 7 rows: one short group
    assert ng < 8
    for kb in (0, 5, rb // 64 - 1):
        for g in range(ng):
            for t in range(4):
                off = r0 * rb + (kb * ng + g) * 64 + t * 16
                assert torch.equal(p[off: off + 16], w[r0 + g, 64 * kb + 16 * t: 64 * kb + 16 * t + 16])


def test_int8_digit_split_is_exact():
    """x * 2^s rounded to 28 bits, cut into base-128 digits d0..d2 in [0,127] and a signed d3:
    sum(q * x) equals the recombined integer dot products exactly."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3584, generator=g) * 3
    q = torch.randint(-127, 128, (16, 3584), generator=g)
    mx = x.abs().max()
    e = int(torch.floor(torch.log2(mx)))
    scale = 2.0 ** (26 - e)
    X = torch.round(x.double() * scale).long()
    assert X.abs().max() < 2 ** 27
    d = [(X >> (7 * i)) & 127 for i in range(3)] + [X >> 21]
    assert d[3].min() >= -64 and d[3].max() <= 63
    assert torch.equal(d[0] + 128 * d[1] + 128 ** 2 * d[2] + 128 ** 3 * d[3], X)
    dots = [(q * di).sum(1) for di in d]
    assert all(int(t.abs().max()) < 2 ** 31 for t in dots)            # fits the s32 accumulator
    exact = (q * X).sum(1)
    assert torch.equal(dots[0] + 128 * dots[1] + 128 ** 2 * dots[2] + 128 ** 3 * dots[3], exact)
    ref = (q.double() * x.double()).sum(1)
    assert ((exact.double() / scale - ref).abs() / ref.abs().clamp_min(1e-3)).max() < 1e-5


def test_bf16_three_piece_split_carries_24_bits():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4096, generator=g) * torch.logspace(-6, 3, 4096)
    p0 = x.to(torch.bfloat16)
    r1 = x - p0.float()
    p1 = r1.to(torch.bfloat16)
    r2 = r1 - p1.float()
    p2 = r2.to(torch.bfloat16)
    err = (p0.float() + p1.float() + p2.float() - x).abs()
    assert (err <= x.abs() * 2.0 ** -23).all()


def test_down_col_slices_are_in_mma_fragment_order():
    """Reading the packed column slices the way the tensor-core instruction reads its first operand
    (lane (g, t): rows g, g + 8; int8: columns 4t..4t+3 and 16+4t..; bf16: per instruction columns 2t, 2t+1
    and 8+2t, 9+2t) reproduces the plain matrix-vector product, summed over the CTAs' slices."""
    import torch
    from megakernels_b200.pack import down_col_range, pack_down_cols
    torch.manual_seed(0)
    n, k, grid = 32, 3584, 148
    tiles = n // 16
    w8 = torch.randint(-127, 128, (n, k), dtype=torch.int8)
    x = torch.randint(-60, 60, (k,), dtype=torch.int64)
    p = pack_down_cols(w8, grid)
    assert p.numel() == grid * tiles * 512
    acc = torch.zeros(n, dtype=torch.int64)
    covered = 0
    for c in range(grid):
        a0, a1 = down_col_range(k, c, grid)
        assert a0 == covered and a1 - a0 <= 32
        covered = a1
        xs = torch.zeros(32, dtype=torch.int64)
        xs[: a1 - a0] = x[a0:a1]
        sl = p[c * tiles * 512: (c + 1) * tiles * 512].view(torch.int8).view(tiles, 32, 4, 4).long()   # [tile][lane][register][byte]
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            lo, hi = xs[4 * t: 4 * t + 4], xs[16 + 4 * t: 16 + 4 * t + 4]
            for tile in range(tiles):
                r = sl[tile, lane]
                acc[tile * 16 + g] += (r[0] * lo).sum() + (r[2] * hi).sum()
                acc[tile * 16 + g + 8] += (r[1] * lo).sum() + (r[3] * hi).sum()
    assert covered == k
    assert torch.equal(acc, w8.long() @ x)
    wb = torch.randn(n, k).to(torch.bfloat16)
    xf = torch.randn(k, dtype=torch.float64)
    p = pack_down_cols(wb, grid)
    assert p.numel() == grid * tiles * 1024
    accf = torch.zeros(n, dtype=torch.float64)
    for c in range(grid):
        a0, a1 = down_col_range(k, c, grid)
        xs = torch.zeros(32, dtype=torch.float64)
        xs[: a1 - a0] = xf[a0:a1]
        sl = p[c * tiles * 1024: (c + 1) * tiles * 1024].view(torch.bfloat16).view(tiles, 32, 2, 4, 2).double()   # [tile][lane][instruction][register][element]
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for m in range(2):
                lo, hi = xs[16 * m + 2 * t: 16 * m + 2 * t + 2], xs[16 * m + 8 + 2 * t: 16 * m + 8 + 2 * t + 2]
                for tile in range(tiles):
                    r = sl[tile, lane, m]
                    accf[tile * 16 + g] += (r[0] * lo).sum() + (r[2] * hi).sum()
                    accf[tile * 16 + g + 8] += (r[1] * lo).sum() + (r[3] * hi).sum()
    assert torch.allclose(accf, wb.double() @ xf, atol=1e-9)
