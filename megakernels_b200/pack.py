"""Weight layout of the decode kernel's GEMV: row slices per CTA, 8-row groups, k-block major.

The kernel gives CTA `c` of `grid` the contiguous rows `plan_rows(N, unit, c, grid)` of every
matrix and streams them through shared memory in chunks of `slot_bytes // row_bytes` rows.  Inside a
chunk, rows are taken in groups of up to 8, and a group is stored k-block major: the first 64 bytes
(64 int8 or 32 bf16 weights) of each of its rows, then the second 64 bytes of each row, and so on.
A warp's 128-bit loads then fetch an 8-row x 64-byte tile as one contiguous 512-byte run, laid out
exactly as the tensor-core instruction wants its second operand.  The bytes of a CTA's slice stay
one contiguous span, so a chunk is still a single bulk copy.

The layout depends on the grid size (one CTA per SM), so weights are packed for the device they will
run on.  The reference's packers are geometry-dependent in the same way
(`common/mkcore/pack.py:25-109`); for the 0.8B CUDA kernel the reference needs no packing beyond the
gate/up row interleave (`qwen3.5-0.8b/qwen_mk/engine.py:86,100`), which `engine.py` keeps.
"""

import torch

KBLOCK = 64       # bytes of one row inside a tile
GROUP = 8         # rows per tile


def plan_rows(rows, unit, cta, grid):
    """Rows [r0, r1) of a `rows`-row matrix owned by CTA `cta` (mirrors `mk_plan_rows` in the C ABI)."""
    units = rows // unit
    return (units * cta // grid) * unit, (units * (cta + 1) // grid) * unit


def _groups(n_rows, rows_per_chunk):
    """(start, size) of every row group of a slice of `n_rows` rows."""
    out = []
    for base in range(0, n_rows, rows_per_chunk):
        nr = min(rows_per_chunk, n_rows - base)
        for g0 in range(0, nr, GROUP):
            out.append((base + g0, min(GROUP, nr - g0)))
    return out


def pack_rows(w, unit, grid, slot_bytes):
    """[N, row_bytes] uint8 (row-major weights as bytes) -> same shape, kernel layout."""
    assert w.dtype == torch.uint8 and w.dim() == 2
    n, rb = w.shape
    assert rb % KBLOCK == 0 and slot_bytes >= rb
    rpc = slot_bytes // rb
    out = torch.empty_like(w)
    nkb = rb // KBLOCK
    for c in range(grid):
        r0, r1 = plan_rows(n, unit, c, grid)
        if rpc % GROUP == 0:
            # groups are the consecutive 8-row blocks of the slice, the last one possibly short
            nfull = (r1 - r0) // GROUP
            if nfull:
                blk = w[r0: r0 + nfull * GROUP].view(nfull, GROUP, nkb, KBLOCK)
                out[r0: r0 + nfull * GROUP] = blk.transpose(1, 2).reshape(nfull * GROUP, rb)
            tail = r0 + nfull * GROUP
            if tail < r1:
                out[tail: r1] = w[tail: r1].view(r1 - tail, nkb, KBLOCK).transpose(0, 1).reshape(r1 - tail, rb)
        else:
            for g0, ng in _groups(r1 - r0, rpc):
                a = r0 + g0
                out[a: a + ng] = w[a: a + ng].view(ng, nkb, KBLOCK).transpose(0, 1).reshape(ng, rb)
    return out


def unpack_rows(p, unit, grid, slot_bytes):
    """Inverse of `pack_rows` (tests, and reading a row back out of a packed matrix)."""
    n, rb = p.shape
    rpc = slot_bytes // rb
    nkb = rb // KBLOCK
    out = torch.empty_like(p)
    for c in range(grid):
        r0, r1 = plan_rows(n, unit, c, grid)
        for g0, ng in _groups(r1 - r0, rpc):
            a = r0 + g0
            out[a: a + ng] = p[a: a + ng].reshape(nkb, ng, KBLOCK).transpose(0, 1).reshape(ng, rb)
    return out


def as_bytes(w):
    """Row-major weight matrix (int8 or bf16) viewed as [N, row_bytes] uint8."""
    w = w.contiguous()
    return w.view(torch.uint8).view(w.shape[0], -1)


# ---- column slices in tensor-core fragment order (the down-projection of the single-sequence kernel) ----
# The CTA that computes SwiGLU outputs [a0, a1) multiplies them right away with columns [a0, a1) of the
# down-projection and publishes 1024 partial sums, so it needs a column slice of the matrix, padded to
# 32 columns.  The slice is stored as 16-row tiles in the order the MMA reads its first operand, one
# 128-bit load per lane and instruction.
DOWN_K = 32       # columns per slice, padded


def down_col_range(inter, cta, grid):
    """SwiGLU outputs [a0, a1) that CTA `cta` produces (its gate/up rows are 2*a0 .. 2*a1)."""
    r0, r1 = plan_rows(2 * inter, 2, cta, grid)
    return r0 // 2, r1 // 2


def _fragment_tiles(sl):
    """[N, kpad] int8 (kpad 32) or bf16 (kpad 16 or 32) -> bytes of its 16-row tiles in fragment order.

    int8 (mma m16n8k32): lane (g, t) of a tile holds rows g and g + 8, columns 4t..4t+3 and 16+4t..16+4t+3,
    as four 32-bit registers [row g | row g + 8] x [low columns | high columns] -> 16 bytes per lane.
    bf16 (one mma m16n8k16 per 16 columns): per instruction rows g, g + 8 and columns 2t, 2t+1 and 8+2t,
    9+2t of its 16 columns -> 16 bytes per lane and instruction, a tile's instructions back to back."""
    n, kpad = sl.shape
    tiles = n // 16
    if sl.dtype == torch.int8:
        assert kpad == 32
        # [tile][hi][g][khalf][t][byte] -> [tile][g][t][khalf][hi][byte]
        x = sl.view(tiles, 2, 8, 2, 4, 4).permute(0, 2, 4, 3, 1, 5)
    else:
        assert sl.dtype == torch.bfloat16 and kpad % 16 == 0
        # [tile][hi][g][mma][khalf][t][elem] -> [tile][g][t][mma][khalf][hi][elem]
        x = sl.view(tiles, 2, 8, kpad // 16, 2, 4, 2).permute(0, 2, 5, 3, 4, 1, 6)
    return x.contiguous().view(torch.uint8).reshape(-1)


def pack_col_slices(w, ranges, kpad):
    """Column slices [a0, a1) of `w` ([N, K] int8 or bf16), each zero-padded to `kpad` columns and stored as
    N / 16 tiles in fragment order, one slice after the other."""
    n = w.shape[0]
    assert n % 16 == 0
    out = []
    for a0, a1 in ranges:
        assert 0 < a1 - a0 <= kpad
        sl = torch.zeros(n, kpad, dtype=w.dtype, device=w.device)
        sl[:, : a1 - a0] = w[:, a0:a1]
        out.append(_fragment_tiles(sl))
    return torch.cat(out)


def pack_down_cols(w, grid):
    """Down-projection [N, K]: per CTA the columns of the SwiGLU outputs it produces, padded to 32."""
    return pack_col_slices(w, [down_col_range(w.shape[1], c, grid) for c in range(grid)], DOWN_K)


def pack_out_cols(w, tasks, cols):
    """DeltaNet out-projection [N, tasks * cols]: per recurrence task the `cols` value columns it owns
    (int8: padded to the 32 columns of one integer MMA; bf16: exactly one 16-column MMA)."""
    kpad = DOWN_K if w.dtype == torch.int8 else cols
    return pack_col_slices(w, [(t * cols, (t + 1) * cols) for t in range(tasks)], kpad)
