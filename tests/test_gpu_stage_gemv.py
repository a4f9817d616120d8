"""The stage machine's GEMV stage through the C ABI (`mk_stage_launch`), one small program per case, against
fp64 matrix products of the dequantised weights: four weight formats, K splits, both prologues, the four
epilogues, ragged row counts, every batch size."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from megakernels_b200.stage import desc as D
from megakernels_b200.stage import pack as P
from megakernels_b200.stage import quant as Q
from megakernels_b200.stage.runtime import Program, Runtime


def _weights(fmt, N, K, seed, block=False):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    kw, rs = {}, None
    if fmt == P.FMT_BF16:
        deq, wq = w.float(), w
    elif fmt == P.FMT_MXFP4:
        pk, sc = Q.quantize_mxfp4(w)
        deq, wq, kw = Q.dequantize_mxfp4(pk, sc).float(), Q.mxfp4_codes(pk), dict(scales=sc)
    elif fmt == P.FMT_FP8 and block:
        wq, bs = Q.quantize_fp8_block(w)
        deq, kw = Q.dequantize_fp8_block(wq, bs), dict(block_scales=bs)
    elif fmt == P.FMT_FP8:
        wq, s = Q.quantize_fp8_row(w)
        deq, rs = Q.dequantize_fp8_row(wq, s), s.float().contiguous()
    else:
        wq, s = Q.quantize_int8_row(w)
        deq, rs = wq.float() * s[:, None], s.float().contiguous()
    return wq, kw, rs, deq.double()


def _run(fmt, N, K, M, splits, *, block=False, prologue="plain", epilogue="store", seed=0, softcap=0.0, act="silu"):
    dev = torch.device("cuda", 0)
    grid = torch.cuda.get_device_properties(dev).multi_processor_count
    glu = epilogue == "glu"
    rows = 2 * N if glu else N
    wq, kw, rs, deq = _weights(fmt, rows, K, seed, block)
    order = P.glu_row_order(N) if glu else None
    packed, meta = P.pack_matrix(fmt, splits, wq, row_order=order, **kw)
    if rs is not None and order is not None:
        rs = rs[order.cuda()].contiguous()
    if rs is not None and rs.numel() < meta["tiles"] * 16:
        rs = torch.cat([rs, torch.zeros(meta["tiles"] * 16 - rs.numel(), device=dev)])
    g = torch.Generator().manual_seed(seed + 1)
    x = (torch.randn(M, K, generator=g) * 1.5).cuda()
    pr = Program(dev, M, grid)
    # every program opens with the embedding stage; here it fills a buffer nothing reads
    pr.embed(pr.zeros(4, 256, dtype=torch.bfloat16), pr.zeros(M, 256), pr.zeros(M, 16), None, 256, 4, keys_valid=False)
    xb = pr.hold(x.clone())
    packed = pr.hold(packed)
    if rs is not None:
        rs = pr.hold(rs)
    out_w = N
    out = pr.zeros(M, out_w)
    args = dict(x_stride=K, out_stride=out_w, n_valid=N, row_scale=rs)
    want_in = x.to(torch.bfloat16).double()
    if prologue == "norm":
        nw = pr.hold((torch.randn(K, generator=g) * 0.1).cuda())
        ssq = pr.hold((x.double() ** 2).reshape(M, K // 16, 16).sum(-1).float())
        args.update(prologue=D.MKS_P_NORM, x_ssq=ssq, norm_w=nw, norm_off=1.0, eps=1e-6, k_total=K)
        xn = x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-6) * (1.0 + nw.double())
        want_in = xn.float().to(torch.bfloat16).double()
    y = want_in @ deq.t()                                    # [M, rows]
    keys = ssq_out = None
    if epilogue == "resid":
        base = (torch.randn(M, N, generator=g)).cuda()
        out.copy_(base)
        ssq_out = pr.zeros(M, N // 16)
        args.update(epilogue=D.MKS_E_RESID, out_ssq=ssq_out)
        want = base.double() + y
    elif glu:
        gt, up = y[:, :N], y[:, N:]
        a = gt * torch.sigmoid(gt) if act == "silu" else torch.nn.functional.gelu(gt, approximate="tanh")
        want = a * up
        args.update(epilogue=D.MKS_E_GLU, act=D.MKS_ACT_SILU if act == "silu" else D.MKS_ACT_GELU_TANH)
    elif epilogue == "logits":
        keys = pr.zeros(M, grid, dtype=torch.int64)
        args.update(epilogue=D.MKS_E_LOGITS, keys=keys, softcap=softcap, row_base=0)
        want = softcap * torch.tanh(y / softcap) if softcap else y
    else:
        want = y
    pr.gemv("t", packed, meta, xb, out, **args)
    rt = Runtime(pr, spin_limit_ms=1000)
    rt.launch(1)
    torch.cuda.synchronize()
    rt.check()
    return out, want, ssq_out, keys, rt


FORMATS = [(P.FMT_BF16, False), (P.FMT_MXFP4, False), (P.FMT_FP8, False), (P.FMT_FP8, True), (P.FMT_INT8, False)]
IDS = ["bf16", "mxfp4", "fp8row", "fp8block", "int8"]


def _tol(want):
    return 2e-3 * float(want.abs().max()) + 1e-4


@pytest.mark.parametrize("fmt,block", FORMATS, ids=IDS)
@pytest.mark.parametrize("M", [1, 2, 5, 8])
def test_store_matches_the_dequantised_product(fmt, block, M):
    out, want, *_ = _run(fmt, 1024, 2048, M, 2, block=block)
    assert float((out.double() - want).abs().max()) <= _tol(want)


@pytest.mark.parametrize("fmt,block", FORMATS, ids=IDS)
@pytest.mark.parametrize("splits", [2, 4, 16])
def test_k_splits_sum_to_the_same_rows(fmt, block, splits):
    out, want, *_ = _run(fmt, 512, 4096, 3, splits, block=block, seed=3)
    assert float((out.double() - want).abs().max()) <= _tol(want)


@pytest.mark.parametrize("fmt,block", FORMATS, ids=IDS)
def test_norm_prologue_and_residual_epilogue(fmt, block):
    out, want, ssq, _, _ = _run(fmt, 1024, 1024, 4, 2, block=block, prologue="norm", epilogue="resid", seed=5)
    assert float((out.double() - want).abs().max()) <= _tol(want)
    # the sums of squares the next stage's RMSNorm reads: one per 16 output rows, of the values just stored
    ref = (out.double() ** 2).reshape(4, -1, 16).sum(-1)
    assert torch.allclose(ssq.double(), ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("fmt,block", FORMATS, ids=IDS)
@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_glu_epilogue(fmt, block, act):
    out, want, *_ = _run(fmt, 768, 1024, 2, 2, block=block, prologue="norm", epilogue="glu", act=act, seed=7)
    assert float((out.double() - want).abs().max()) <= _tol(want) + 1e-3 * float(want.abs().max())


@pytest.mark.parametrize("softcap", [0.0, 30.0])
def test_logits_epilogue_writes_the_argmax_keys(softcap):
    N = 5000                                            # ragged: the last tile has 8 valid rows
    out, want, _, keys, _ = _run(P.FMT_BF16, N, 1024, 3, 1, epilogue="logits", softcap=softcap, seed=9)
    assert float((out.double() - want).abs().max()) <= _tol(want)
    # key = order-preserving image of the score in the high word, ~row in the low word, compared unsigned
    best = (keys ^ (-2 ** 63)).max(dim=1).values
    ids = (0xFFFFFFFF - (best & 0xFFFFFFFF)).long()
    top = out.argmax(-1)
    assert torch.equal(ids.cpu(), top.cpu())


def test_ragged_rows_leave_the_padding_untouched():
    out, want, *_ = _run(P.FMT_MXFP4, 1000, 1024, 2, 2, seed=11)
    assert out.shape[1] == 1000
    assert float((out.double() - want).abs().max()) <= _tol(want)


def test_a_stage_runs_twice_with_the_same_counters():
    """Partial-tile counters return to zero, so the same program can be launched again."""
    out, want, _, _, rt = _run(P.FMT_FP8, 512, 4096, 2, 8, seed=13)
    assert float((out.double() - want).abs().max()) <= _tol(want)
    first = out.clone()
    out.zero_()
    rt.launch(1)
    torch.cuda.synchronize()
    rt.check()
    assert torch.equal(out, first)
