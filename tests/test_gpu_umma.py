"""The block-scaled tcgen05 GEMV against a float64 product of the dequantised weights.

Two references: (a) the product with the kernel's own digit planes of x (`umma.digit_planes`, exact sums of e2m1
digits): the tensor core multiplies exactly and adds in fp32, so the difference is accumulation order only, 2e-5 of
sum |w||x|; (b) the product with bf16(x), what the reference decoders compute: the planes drop what lies more than
2 * pieces bits below a 32-column block's largest value, 1e-3 of sum |w||x| at six planes."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from megakernels_b200.stage import quant as Q
from megakernels_b200.stage import umma as U


def make(rows, k, batch, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(rows, k, generator=g, device="cuda") * 0.02
    packed, scales = Q.quantize_mxfp4(w)
    x = torch.randn(batch, k, generator=g, device="cuda") * torch.logspace(-2, 1, k, device="cuda")[torch.randperm(k, generator=g, device="cuda")]
    return packed, scales, Q.dequantize_mxfp4(packed, scales).double(), x.contiguous()


@pytest.mark.parametrize("rows,k,batch,splits,pieces", [
    (128, 128, 1, 1, 6), (256, 256, 8, 1, 6), (1000, 1024, 3, 2, 4), (5120, 5120, 8, 1, 6), (4096, 17408, 8, 4, 6),
    (34816, 5120, 1, 1, 8), (34816, 5120, 8, 1, 6)])
def test_gemv_matches_the_dequantised_product(rows, k, batch, splits, pieces):
    packed, scales, wd, x = make(rows, k, batch, rows + k + batch)
    op = U.Gemv(packed, scales, splits=splits, pieces=pieces)
    got = op(x).double()
    torch.cuda.synchronize()
    op.check()
    digits, exps = U.digit_planes(x, pieces)
    exact = U.planes_value(digits, exps) @ wd.t()
    ref = x.to(torch.bfloat16).double() @ wd.t()
    bound = x.to(torch.bfloat16).double().abs() @ wd.abs().t()
    assert float(((got - exact).abs() / bound).max()) < 2e-5
    assert float(((got - ref).abs() / bound).max()) < (1e-3 if pieces >= 6 else 2e-2)
    assert int(op.cnt.abs().max()) == 0
    # a second launch on the same buffers gives the same bits (the partial tiles are added in a fixed order)
    again = op(x)
    torch.cuda.synchronize()
    assert torch.equal(again.double(), got)


def test_unrounded_inputs_and_zero_blocks():
    packed, scales, wd, x = make(384, 512, 2, 5)
    x[0, 64:96] = 0.0
    x[1] = 0.0
    op = U.Gemv(packed, scales, pieces=8)
    got = op(x, round_bf16=False).double()
    torch.cuda.synchronize()
    op.check()
    bound = x.double().abs() @ wd.abs().t()
    assert float((got[0] - x[0].double() @ wd.t()).abs().max() / bound[0].max()) < 1e-4
    assert float(got[1].abs().max()) == 0.0
