"""Weight formats of the large shapes: MXFP4, FP8 with 128 x 128 block scales, FP8 with row scales.

The reference consumes vendor checkpoints that are already quantised and only dequantises them
(`qwen3.8-27b-gfx942/mk/reference.py:40-59,76-83` for MXFP4, `qwen3.6-35b-a3b-gfx942/mk/reference.py:55-58`
for FP8 blocks, `gemma4-26b-a4b-gfx942/mk/reference.py:150-157` for FP8 rows).  No checkpoint is available
where this library is tested, so these functions *produce* the same formats from seeded bf16 weights;
the tests pin them by a round trip through the reference's dequantisers.
"""

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)      # code -> magnitude; bit 3 of a code is the sign
_E2M1_MID = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)         # rounding boundaries between neighbouring magnitudes


def quantize_mxfp4(w):
    """[N, K] -> (codes uint8 [N, K/2], low nibble = even k; scales uint8 [N, K/32], e8m0: 2^(s - 127)).

    Per group of 32: the scale is the power of two that brings the largest magnitude into e2m1's top
    binade (4..6], values round to the nearest e2m1 magnitude (boundaries go to the even code) and
    saturate at 6; -0 is stored as +0, as the reference's packer canonicalises it (`common/mkcore/fp4.py:14,37`)."""
    N, K = w.shape
    assert K % 32 == 0
    x = w.float().reshape(N, K // 32, 32)
    amax = x.abs().amax(-1, keepdim=True)
    e = torch.floor(torch.log2(amax.clamp_min(2.0 ** -120))) - 2.0
    e = torch.where(amax > 0, e, torch.zeros_like(e)).clamp(-127, 127)
    v = x / torch.exp2(e)
    mag = v.abs().clamp_max(6.0)
    mid = torch.tensor(_E2M1_MID, device=w.device)
    code = torch.bucketize(mag, mid, right=False)            # boundary values fall to the lower code ...
    tie_up = torch.zeros_like(code, dtype=torch.bool)
    for i, m in enumerate(_E2M1_MID):                         # ... unless the lower code is odd (round half to even)
        tie_up |= (mag == m) & (i % 2 == 1)
    code = (code + tie_up.to(code.dtype)).to(torch.uint8)
    sign = ((v < 0) & (code > 0)).to(torch.uint8) << 3
    code = (code | sign).reshape(N, K)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    scales = (e.squeeze(-1) + 127).to(torch.uint8)
    return packed.contiguous(), scales.contiguous()


def dequantize_mxfp4(packed, scales):
    """Inverse of `quantize_mxfp4`: bf16 [N, K] (exact, every product fits bf16)."""
    lut = torch.tensor(E2M1_VALUES + tuple(-x for x in E2M1_VALUES), device=packed.device)
    lo, hi = lut[(packed & 0xF).long()], lut[(packed >> 4).long()]
    w = torch.stack([lo, hi], dim=-1).reshape(packed.shape[0], -1)
    return (w * torch.exp2(scales.float() - 127.0).repeat_interleave(32, dim=1)).to(torch.bfloat16)


def mxfp4_codes(packed):
    """[N, K/2] packed bytes -> one code per element [N, K] (uint8)."""
    return torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(packed.shape[0], -1)


FP8_MAX = 448.0


def quantize_fp8_block(w, block=128):
    """[N, K] -> (e4m3fn [N, K], bf16 scales [ceil(N/128), ceil(K/128)]): w ~ fp8 * scale of its 128 x 128 block."""
    N, K = w.shape
    nb, kb = -(-N // block), -(-K // block)
    x = torch.zeros(nb * block, kb * block, device=w.device)
    x[:N, :K] = w.float()
    amax = x.reshape(nb, block, kb, block).abs().amax(dim=(1, 3))
    scale = (amax / FP8_MAX).clamp_min(1e-12).to(torch.bfloat16)
    full = scale.float().repeat_interleave(block, 0).repeat_interleave(block, 1)[:N, :K]
    q = (w.float() / full).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def dequantize_fp8_block(q, scale, block=128):
    full = scale.float().repeat_interleave(block, -2).repeat_interleave(block, -1)
    return q.float() * full[..., : q.shape[-2], : q.shape[-1]]


def quantize_fp8_row(w):
    """[N, K] -> (e4m3fn [N, K], bf16 scale per output row [N]): y = (x @ q^T) * scale."""
    amax = w.float().abs().amax(dim=1)
    scale = (amax / FP8_MAX).clamp_min(1e-12).to(torch.bfloat16)
    q = (w.float() / scale.float()[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def dequantize_fp8_row(q, scale):
    return q.float() * scale.float()[:, None]


def quantize_int8_row(w):
    """[N, K] -> (int8 [N, K], fp32 scale per row): symmetric, scale = absmax / 127."""
    amax = w.float().abs().amax(dim=1)
    scale = (amax / 127.0).clamp_min(1e-12)
    q = torch.round(w.float() / scale[:, None]).clamp(-127, 127).to(torch.int8)
    return q, scale
