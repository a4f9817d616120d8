"""Quantisers and tile packers of the large-shape engines (CPU): round trips, the lane walk the kernel
performs, and equality with the reference's own MXFP4 dequantiser when its checkout is present."""

import os
import sys

import pytest
import torch

from megakernels_b200.stage import pack as P
from megakernels_b200.stage import quant as Q

REFERENCE = os.environ.get("MK_REFERENCE_ROOT",
                           os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))


def _w(n, k, seed=0, sd=0.05):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, k, generator=g) * sd).to(torch.bfloat16)


def test_mxfp4_values_and_scales():
    w = _w(48, 256)
    pk, sc = Q.quantize_mxfp4(w)
    assert pk.shape == (48, 128) and sc.shape == (48, 8) and pk.dtype == sc.dtype == torch.uint8
    deq = Q.dequantize_mxfp4(pk, sc).float()
    # every group's largest magnitude lands in the top binade, so the error is at most half a step of that binade
    grp = w.float().reshape(48, 8, 32)
    err = (deq.reshape(48, 8, 32) - grp).abs().amax(-1)
    assert bool((err <= grp.abs().amax(-1) * 0.25 + 1e-12).all())
    # quantising a dequantised matrix is the identity on the codes (idempotence)
    pk2, sc2 = Q.quantize_mxfp4(deq.to(torch.bfloat16))
    assert torch.equal(Q.dequantize_mxfp4(pk2, sc2), deq.to(torch.bfloat16))
    # no negative zero codes
    codes = Q.mxfp4_codes(pk)
    assert not bool((codes == 8).any())


def test_mxfp4_of_zeros_and_extremes():
    w = torch.zeros(16, 64, dtype=torch.bfloat16)
    w[0, 0], w[1, 5] = 3.0e4, -1e-30
    pk, sc = Q.quantize_mxfp4(w)
    deq = Q.dequantize_mxfp4(pk, sc).float()
    assert torch.isfinite(deq).all() and float(deq[2:].abs().max()) == 0.0
    assert abs(float(deq[0, 0]) - 3.0e4) <= 0.25 * 3.0e4


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "qwen3.8-27b-gfx942")), reason="reference checkout absent")
def test_mxfp4_dequantiser_equals_the_reference():
    sys.path.insert(0, os.path.join(REFERENCE, "qwen3.8-27b-gfx942"))
    for k in [k for k in sys.modules if k == "mk" or k.startswith("mk.")]:
        del sys.modules[k]                      # another model's `mk` package may have been imported by an earlier test
    from mk import reference as R
    pk, sc = Q.quantize_mxfp4(_w(64, 512, seed=3))
    assert torch.equal(Q.dequantize_mxfp4(pk, sc), R.dequant_mxfp4(pk, sc))
    g = torch.Generator().manual_seed(1)
    pk = torch.randint(0, 256, (32, 64), generator=g, dtype=torch.uint8)
    sc = torch.randint(100, 140, (32, 4), generator=g, dtype=torch.uint8)
    assert torch.equal(Q.dequantize_mxfp4(pk, sc).float(), R.dequant_mxfp4(pk, sc).float())


def test_fp8_and_int8_quantisers_round_trip():
    w = _w(200, 384, seed=2)
    q, s = Q.quantize_fp8_block(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 3)
    assert float((Q.dequantize_fp8_block(q, s) - w.float()).abs().max()) <= float(w.float().abs().max()) * 0.07
    q, s = Q.quantize_fp8_row(w)
    assert float((Q.dequantize_fp8_row(q, s) - w.float()).abs().max()) <= float(w.float().abs().max()) * 0.07
    q, s = Q.quantize_int8_row(w)
    assert q.dtype == torch.int8 and float((q.float() * s[:, None] - w.float()).abs().max()) <= float(s.max()) * 0.5 + 1e-9


@pytest.mark.parametrize("fmt", [P.FMT_BF16, P.FMT_MXFP4, P.FMT_FP8, P.FMT_INT8])
@pytest.mark.parametrize("splits", [1, 2])
def test_packed_tiles_read_back_lane_by_lane(fmt, splits):
    """`unpack_matrix` walks a packed matrix exactly as the kernel's lanes do; it must return the matrix."""
    N, K = 40, 256                                      # ragged: 2.5 tiles
    w = _w(N, K, seed=4)
    kw = {}
    if fmt == P.FMT_BF16:
        src, want = w, w.float()
    elif fmt == P.FMT_MXFP4:
        pk, sc = Q.quantize_mxfp4(w)
        src, kw = Q.mxfp4_codes(pk), dict(scales=sc)
        lut = torch.tensor(Q.E2M1_VALUES + tuple(-x for x in Q.E2M1_VALUES))
        want = lut[src.long()]
    elif fmt == P.FMT_FP8:
        src, _ = Q.quantize_fp8_row(w)
        want = src.float()
    else:
        src, _ = Q.quantize_int8_row(w)
        want = src.float()
    packed, meta = P.pack_matrix(fmt, splits, src, **kw)
    assert meta["tiles"] == 3 and meta["splits"] == splits and meta["kc"] == K // splits
    assert packed.numel() == meta["bytes"] == 3 * splits * (meta["unit_steps"] // meta["chunk_steps"]) * meta["chunk_bytes"]
    assert meta["chunk_bytes"] <= P.SLOT_BYTES and meta["chunk_bytes"] % 16 == 0
    back = P.unpack_matrix(packed, meta, K)
    assert torch.equal(back[:N], want)
    assert float(back[N:].abs().max()) == 0.0


def test_glu_row_order_pairs_gate_and_up_rows():
    order = P.glu_row_order(24)
    assert order.tolist()[:16] == list(range(8)) + list(range(24, 32))
    assert sorted(order.tolist()) == list(range(48))


def test_chunk_geometry():
    for us in (4, 8, 12, 20, 80):
        cs = P.pick_chunk_steps(us, P.FMT_MXFP4)
        assert us % cs == 0 and P.chunk_bytes(P.FMT_MXFP4, cs) <= P.SLOT_BYTES
    assert P.pick_chunk_steps(12, P.FMT_FP8, block_scaled=True) % 4 == 0
    assert P.chunk_bytes(P.FMT_MXFP4, 8) == 8 * 512 + 8 * 32
    assert P.chunk_bytes(P.FMT_FP8, 8, True) == 8 * 512 + 16
