"""Weight-only quantisers for the decode kernel.

int8 per output channel: one fp32 scale per row, `scale = absmax(row) * fl32(1/127)`, symmetric,
`q = round(w / scale)` in [-127, 127].  The kernel stores `q + 128` as an unsigned byte so that
a byte-permute can splice it into the mantissa of 2^23 and one subtraction recovers `q` exactly.

The reference's int8 format is Q8_0 instead: one bf16 scale per 32 weights appended to each row
(`qwen3.5-0.8b/qwen_mk/engine.py:25-46`).  The per-channel form here follows the benchmark
configuration this library is measured on; the calling convention is the same: quantise, hand
the packed bytes to the kernel, and check the kernel against a decoder that runs on the
*dequantised* weights (`qwen3.5-0.8b/tests/test_int8.py:25-35`).
"""

import torch

INV_127 = float(torch.tensor(1.0 / 127.0, dtype=torch.float32))
ROW_SLICE = 16384  # rows per pass, so the LM head never needs a multi-GB fp32 temporary


def quantize_int8_rows(w):
    """[R, K] float/bf16 -> (uint8 [R, K] holding q + 128, float32 [R] scales)."""
    R, K = w.shape
    q = torch.empty(R, K, dtype=torch.uint8, device=w.device)
    scale = torch.empty(R, dtype=torch.float32, device=w.device)
    for r in range(0, R, ROW_SLICE):
        blk = w[r: r + ROW_SLICE].float()
        # absmax * fl(1/127), not absmax / 127: CUDA kernels turn a division by a scalar into a
        # multiplication by its reciprocal, and the scales must not depend on the device
        s = (blk.abs().amax(dim=1) * INV_127).clamp_min(1e-12)
        scale[r: r + ROW_SLICE] = s
        q[r: r + ROW_SLICE] = (torch.round(blk / s[:, None]).clamp_(-127, 127) + 128).to(torch.uint8)
    return q, scale


def dequantize_int8_rows(q, scale):
    """Inverse of `quantize_int8_rows`, in fp32: (byte - 128) * scale[row]."""
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    for r in range(0, q.shape[0], ROW_SLICE):
        out[r: r + ROW_SLICE] = (q[r: r + ROW_SLICE].to(torch.int16) - 128).float() * scale[r: r + ROW_SLICE, None]
    return out


def roundtrip_int8_rows(w):
    """The fp32 weights an int8 kernel effectively uses."""
    return dequantize_int8_rows(*quantize_int8_rows(w))


# Names of the projection matrices that are quantised; norms, conv taps, gates' biases stay bf16.
GEMV_WEIGHTS = ("mlp.gate_proj", "mlp.up_proj", "mlp.down_proj", "linear_attn.in_proj_qkv", "linear_attn.in_proj_z",
                "linear_attn.in_proj_b", "linear_attn.in_proj_a", "linear_attn.out_proj", "self_attn.q_proj",
                "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "fc.weight")


def is_gemv_weight(name):
    return name.endswith(".weight") and any(n in name for n in GEMV_WEIGHTS)


def dequantized_weights(w, quant, embed_int8=True):
    """The weight dict a reference decoder must run on to see what the kernel sees.

    For `quant="int8"` every projection matrix is replaced by its int8 round trip; with
    `embed_int8` the embedding table (and therefore the tied LM head) is too, otherwise only an
    `lm_head.weight` copy is (the reference's choice, `tests/test_int8.py:33`).
    """
    if quant == "bf16":
        return dict(w)
    assert quant == "int8", quant
    out = {}
    for k, v in w.items():
        out[k] = roundtrip_int8_rows(v) if is_gemv_weight(k) else v
    if "embed_tokens.weight" in w:
        rt = roundtrip_int8_rows(w["embed_tokens.weight"])
        if embed_int8:
            out["embed_tokens.weight"] = rt
        else:
            out["lm_head.weight"] = rt
    if "lm_head.weight" in w:
        out["lm_head.weight"] = roundtrip_int8_rows(w["lm_head.weight"])
    return out
