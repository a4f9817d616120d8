"""Tile layouts of the stage-machine megakernel's weight stream.

A GEMV matrix [N, K] is cut into units: (K split s, 16-row tile t), stored unit after unit in the order
(s, t).  A unit is a sequence of *tile steps* of 512 bytes: the bytes lane 0..31 of the consuming warp
load with one 128-bit read each.  Lane (g = lane // 4, q = lane % 4) holds 8 bytes of tile row g and
8 bytes of tile row g + 8: the operands of the step's MMAs for input columns
k0 + 16 j + 4 q + {0, 1, 2, 3}, j = 0 .. (64, 32 or 16 columns per step) / 16 - 1.  Steps are grouped
into ring chunks of `chunk_steps`; a chunk carries its scales behind its steps:

    MXFP4   64 columns per step; per step 32 scale bytes [g][half][32-column group] (e8m0)
    FP8     32 columns per step; block-scaled matrices: per 4 steps two fp32 (rows 0-7, rows 8-15 of the tile)
    INT8    32 columns per step
    BF16    16 columns per step

`row_order` permutes matrix rows into tile rows (the GLU layout puts 8 gate rows and their 8 up rows
into one tile, so that one lane holds a gate / up pair).  The reference's AMD tile layouts
(`common/mkcore/fp4.py`, `common/mkcore/pack.py`) serve the same purpose for MFMA fragments.
"""

import torch

FMT_BF16, FMT_MXFP4, FMT_FP8, FMT_INT8 = 0, 1, 2, 3
# Bit positions of the pre-arranged MXFP4 words (scale group 0): register k of a word holds two values, the sign
# of the low one at MXFP4_SIGN_BIT[k], its three magnitude bits from MXFP4_MAG_BIT[k] up; the high one 16 bits higher.
# Register k is rebuilt as ((w << (15 - sign)) & 0x80008000) | ((w << (9 - mag)) & 0x0E000E00).
MXFP4_SIGN_BIT = (15, 12, 14, 13)
MXFP4_MAG_BIT = (9, 6, 3, 0)
STEP_K = {FMT_BF16: 16, FMT_MXFP4: 64, FMT_FP8: 32, FMT_INT8: 32}
SLOT_BYTES = 4352


def pick_chunk_steps(unit_steps, fmt, block_scaled=False):
    for cs in (8, 4, 2, 1):
        if unit_steps % cs == 0 and not (block_scaled and cs % 4):
            return cs
    raise ValueError(f"no chunk size divides {unit_steps} steps")


def chunk_bytes(fmt, cs, block_scaled=False):
    extra = cs * 32 if fmt == FMT_MXFP4 else ((cs // 4) * 8 if block_scaled else 0)
    return (cs * 512 + extra + 15) // 16 * 16


def glu_row_order(n_pairs):
    """Tile-row order of a [gate rows | up rows] matrix with `n_pairs` rows each: tile t holds gate rows
    8t..8t+7 then up rows 8t..8t+7."""
    assert n_pairs % 8 == 0
    t = torch.arange(n_pairs // 8)[:, None, None]
    half = torch.arange(2)[None, :, None]
    g = torch.arange(8)[None, None, :]
    return (half * n_pairs + t * 8 + g).reshape(-1)


def _pad_rows(x, rows):
    if x.shape[0] == rows:
        return x
    out = torch.zeros((rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    out[: x.shape[0]] = x
    return out


def _steps_view(x, splits, step_elems):
    """[T*16, K] -> [T, half, g, S, steps, step_elems]"""
    R, K = x.shape
    kc = K // splits
    return x.reshape(R // 16, 2, 8, splits, kc // step_elems, step_elems)


def pack_matrix(fmt, splits, w, scales=None, block_scales=None, row_order=None):
    """Pack one matrix.  Returns (bytes uint8 [units * unit_bytes], meta dict).

    fmt BF16: w bf16 [N, K].  MXFP4: w = codes uint8 [N, K] (one per element), scales uint8 [N, K/32].
    FP8: w float8_e4m3fn [N, K], block_scales fp32/bf16 [ceil(N/128), ceil(K/128)] or None.  INT8: w int8 [N, K].
    """
    N, K = w.shape
    if row_order is not None:
        w = w[row_order.to(w.device)]
        if scales is not None:
            scales = scales[row_order.to(w.device)]
    T = -(-N // 16)
    step_k = STEP_K[fmt]
    assert K % splits == 0 and (K // splits) % step_k == 0, (K, splits, step_k)
    kc = K // splits
    unit_steps = kc // step_k
    block_scaled = block_scales is not None
    cs = pick_chunk_steps(unit_steps, fmt, block_scaled)
    nch = unit_steps // cs
    cb = chunk_bytes(fmt, cs, block_scaled)
    dev = w.device
    if fmt == FMT_BF16:
        x = _pad_rows(w.contiguous().view(torch.int16), T * 16)
        v = _steps_view(x, splits, 16).reshape(T, 2, 8, splits, unit_steps, 4, 4)          # t h g s st q sl
        body = v.permute(3, 0, 4, 2, 5, 1, 6).contiguous().view(torch.uint8)                 # s t st g q h sl(2 bytes)
        body = body.reshape(splits, T, nch, cs * 512)
        extra = None
    elif fmt == FMT_MXFP4:
        x = _pad_rows(w, T * 16)
        v = _steps_view(x, splits, 64).reshape(T, 2, 8, splits, unit_steps, 4, 4, 2, 2)    # t h g s st j q slp nib
        v = v.permute(3, 0, 4, 2, 6, 1, 5, 7, 8).contiguous()                                # s t st g q h j slp nib
        plain = (v[..., 0] | (v[..., 1] << 4))                                               # s t st g q h j slp: one byte per nibble pair
        # scale group 0 (j = 0, 1) goes out with its bits pre-arranged for shift-and-mask conversion: register
        # k = 2 j + slp of a word takes nib 0 in its low half and nib 1 in its high half
        c = v[..., :2, :, :].to(torch.int64)                                                 # s t st g q h j(2) slp nib
        word = torch.zeros(c.shape[:-3], dtype=torch.int64, device=c.device)
        for j in range(2):
            for slp in range(2):
                k = 2 * j + slp
                for nib in range(2):
                    code = c[..., j, slp, nib]
                    word |= ((code >> 3) << (MXFP4_SIGN_BIT[k] + 16 * nib)) | ((code & 7) << (MXFP4_MAG_BIT[k] + 16 * nib))
        arranged = torch.stack([(word >> (8 * i)) & 0xFF for i in range(4)], dim=-1).to(torch.uint8)   # s t st g q h 4
        lane = torch.cat([arranged, plain[..., 2:, :].reshape(plain.shape[:-2] + (4,))], dim=-1)       # s t st g q h 8: word of group 0, word of group 1
        # the kernel's 128-bit read is (row g: group 0, group 1, row g + 8: group 0, group 1): h is already outside
        body = lane.reshape(splits, T, nch, cs * 512)
        sc = _pad_rows(scales, T * 16).reshape(T, 2, 8, splits, unit_steps, 2)               # t h g s st grp
        extra = sc.permute(3, 0, 4, 2, 1, 5).contiguous().reshape(splits, T, nch, cs * 32)   # s t st g h grp
    else:
        x = _pad_rows(w.contiguous().view(torch.uint8), T * 16)
        v = _steps_view(x, splits, 32).reshape(T, 2, 8, splits, unit_steps, 2, 4, 4)       # t h g s st j q sl
        body = v.permute(3, 0, 4, 2, 6, 1, 5, 7).contiguous().reshape(splits, T, nch, cs * 512)   # s t st g q h j sl
        extra = None
        if block_scaled:
            assert kc % 128 == 0 and fmt == FMT_FP8
            rows = torch.arange(T * 16, device=dev)
            src_rows = rows if row_order is None else _pad_rows(row_order.to(dev), T * 16)
            src_rows = src_rows.clamp_max(N - 1)
            per_row = block_scales.float()[(src_rows // 128)]                                 # [T*16, K/128]
            per_row = per_row[:, : K // 128].reshape(T, 2, 8, splits, kc // 128)[:, :, 0]     # [T, h, s, blocks]
            extra = per_row.permute(2, 0, 3, 1).contiguous()                                  # s t blk h
            extra = extra.reshape(splits, T, nch, (cs // 4) * 2).view(torch.uint8).reshape(splits, T, nch, (cs // 4) * 8)
    parts = [body] if extra is None else [body, extra]
    used = sum(p.shape[-1] for p in parts)
    if used < cb:
        parts.append(torch.zeros(splits, T, nch, cb - used, dtype=torch.uint8, device=dev))
    out = torch.cat(parts, dim=-1).reshape(-1)
    meta = dict(fmt=fmt, tiles=T, splits=splits, unit_steps=unit_steps, chunk_steps=cs, chunk_bytes=cb, kc=kc, rows=N,
                block_scaled=block_scaled, bytes=out.numel())
    return out, meta


def unpack_matrix(packed, meta, K):
    """Inverse of `pack_matrix` by walking the layout the way the kernel's lanes do (test helper):
    returns (values fp32 [T*16, K] as the MMAs see them *before* scaling, scale bytes or floats)."""
    fmt, T, S, us, cs, cb = meta["fmt"], meta["tiles"], meta["splits"], meta["unit_steps"], meta["chunk_steps"], meta["chunk_bytes"]
    nch = us // cs
    p = packed.reshape(S, T, nch, cb).cpu()
    out = torch.zeros(T * 16, K)
    step_k = STEP_K[fmt]
    kc = meta["kc"]
    lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
    for s in range(S):
        for t in range(T):
            for ch in range(nch):
                blob = p[s, t, ch]
                for st in range(cs):
                    k0 = s * kc + (ch * cs + st) * step_k
                    for lane in range(32):
                        g, q = lane // 4, lane % 4
                        b = blob[st * 512 + lane * 16: st * 512 + lane * 16 + 16]
                        for half in range(2):
                            row = t * 16 + g + 8 * half
                            hb = b[half * 8: half * 8 + 8]
                            if fmt == FMT_MXFP4:
                                word = int.from_bytes(bytes(hb[:4].tolist()), "little")
                                for j in range(2):                                  # scale group 0: pre-arranged bits
                                    for slp in range(2):
                                        r = 2 * j + slp
                                        for nib in range(2):
                                            sgn = (word >> (MXFP4_SIGN_BIT[r] + 16 * nib)) & 1
                                            mag = (word >> (MXFP4_MAG_BIT[r] + 16 * nib)) & 7
                                            out[row, k0 + 16 * j + 4 * q + 2 * slp + nib] = lut[mag | (sgn << 3)]
                                for j in range(2, 4):                               # scale group 1: plain nibbles
                                    for slp in range(2):
                                        byte = int(hb[2 * j + slp])
                                        k = k0 + 16 * j + 4 * q + 2 * slp
                                        out[row, k] = lut[byte & 0xF]
                                        out[row, k + 1] = lut[byte >> 4]
                            elif fmt == FMT_BF16:
                                vals = hb.view(torch.bfloat16).float()
                                out[row, k0 + 4 * q: k0 + 4 * q + 4] = vals
                            else:
                                for j in range(2):
                                    raw = hb[4 * j: 4 * j + 4]
                                    vals = raw.view(torch.float8_e4m3fn).float() if fmt == FMT_FP8 else raw.view(torch.int8).float()
                                    out[row, k0 + 16 * j + 4 * q: k0 + 16 * j + 4 * q + 4] = vals
    return out
