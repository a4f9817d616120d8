"""Host side of the block-scaled tcgen05 GEMV for MXFP4 weights (`include/mk_umma.h`).

`pack(packed, scales, splits)` turns the row-major MXFP4 arrays of `quant.quantize_mxfp4` into the chunked layout the
kernel streams (128 rows x 128 columns per chunk, already in the tensor core's shared-memory order, each chunk
followed by its scale atom); `Gemv` owns the scratch buffers of one matrix and launches the kernel;
`digit_planes` is the kernel's input decomposition restated in torch (what the B operand holds), so the tests can
separate "the planes are wrong" from "the MMA is wrong".

The reference's counterpart is the dequantising GEMV of its 27B engine (`common/mkcore/gemv.py:48-52` with the
MXFP4 tables of `qwen3.8-27b-gfx942/mk/reference.py:40-83`)."""

import ctypes
import os

import torch

from .. import _lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "include", "mk_umma.h")
ROWS, CHUNK_K, CHUNK_BYTES, MAX_SLICE_K, MAX_SPLITS = 128, 128, 8704, 5120, 8
UMMA_EXPORTS = ["mk_umma_gemv", "mk_umma_scratch_bytes"]


class UmmaArgs(ctypes.Structure):
    _fields_ = [("w", ctypes.c_uint64), ("x", ctypes.c_uint64), ("out", ctypes.c_uint64), ("part", ctypes.c_uint64),
                ("cnt", ctypes.c_uint64), ("status", ctypes.c_uint64), ("stream", ctypes.c_uint64),
                ("prof", ctypes.c_uint64), ("spin_limit_ns", ctypes.c_int64),
                ("rows", ctypes.c_int32), ("k", ctypes.c_int32), ("batch", ctypes.c_int32), ("pieces", ctypes.c_int32),
                ("splits", ctypes.c_int32), ("device", ctypes.c_int32), ("round_bf16", ctypes.c_int32), ("grid", ctypes.c_int32)]


_bound = False


def lib():
    global _bound
    L = _lib.load()
    if not _bound:
        L.mk_umma_gemv.argtypes = [ctypes.POINTER(UmmaArgs)]
        L.mk_umma_gemv.restype = ctypes.c_int
        L.mk_umma_scratch_bytes.argtypes = [ctypes.c_int] * 6
        L.mk_umma_scratch_bytes.restype = ctypes.c_int64
        _bound = True
    return L


def pack(packed, scales, splits=1):
    """packed uint8 [rows, k/2] (even column in the low nibble), scales uint8 [rows, k/32]  ->  uint8
    [splits, row_blocks, chunks_per_split, 8704].  Rows are padded with zeros to a multiple of 128."""
    rows, k = packed.shape[0], packed.shape[1] * 2
    if k % (splits * CHUNK_K):
        raise ValueError(f"k = {k} is not {splits} slices of whole {CHUNK_K}-column chunks")
    rb = (rows + ROWS - 1) // ROWS
    pad = rb * ROWS - rows
    if pad:
        packed = torch.cat([packed, packed.new_zeros(pad, packed.shape[1])])
        scales = torch.cat([scales, scales.new_full((pad, scales.shape[1]), 127)])
    kc = k // CHUNK_K
    # data: [rb, 16 row groups, 8 rows, kc, 4 cores, 16 bytes] -> [rb, kc, 16, 4, 8, 16]
    d = packed.reshape(rb, 16, 8, kc, 4, 16).permute(0, 3, 1, 4, 2, 5).reshape(rb, kc, 8192)
    # scale atom: byte (row % 32) * 16 + (row / 32) * 4 + block: [rb, 4 (row / 32), 32 (row % 32), kc, 4] -> [rb, kc, 32, 4, 4]
    s = scales.reshape(rb, 4, 32, kc, 4).permute(0, 3, 2, 1, 4).reshape(rb, kc, 512)
    chunks = torch.cat([d, s], dim=-1)                                             # [rb, kc, 8704]
    cps = kc // splits
    return chunks.reshape(rb, splits, cps, CHUNK_BYTES).permute(1, 0, 2, 3).contiguous()


def unpack(chunks, rows):
    """Inverse of `pack`: [splits, row_blocks, chunks_per_split, 8704] -> (packed [rows, k/2], scales [rows, k/32])."""
    splits, rb, cps, _ = chunks.shape
    kc = splits * cps
    c = chunks.permute(1, 0, 2, 3).reshape(rb, kc, CHUNK_BYTES)
    d = c[..., :8192].reshape(rb, kc, 16, 4, 8, 16).permute(0, 2, 4, 1, 3, 5).reshape(rb * ROWS, kc * 64)
    s = c[..., 8192:].reshape(rb, kc, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(rb * ROWS, kc * 4)
    return d[:rows].contiguous(), s[:rows].contiguous()


def digit_planes(x, pieces, round_bf16=True):
    """The kernel's decomposition of the inputs, in torch: x [batch, k] -> (digits int [pieces, batch, k] in -3..3,
    exponents int [pieces, batch, k/32]) with x ~ sum_p digits[p] * 0.5 * 2^exponents[p]."""
    v = x.float()
    if round_bf16:
        v = v.to(torch.bfloat16).float()
    B, K = v.shape
    blk = v.reshape(B, K // 32, 32)
    mx = blk.abs().amax(-1)
    e = (mx.view(torch.int32) >> 23) - 127
    live = (mx > 0) & (e >= -100) & (e <= 100)
    e = torch.where(live, e, torch.zeros_like(e))
    q = torch.round(blk.abs().double() * torch.exp2((2 * pieces - 1 - e).double())[..., None]).clamp_max(4 ** pieces - 1).long()
    q = torch.where(live[..., None], q, torch.zeros_like(q))
    sign = torch.where(blk < 0, -1, 1)
    digits = torch.stack([((q >> (2 * p)) & 3) * sign for p in range(pieces)]).reshape(pieces, B, K)
    exps = torch.stack([e + 2 - 2 * pieces + 2 * p for p in range(pieces)])
    return digits, exps


def planes_value(digits, exps):
    """What the digit planes add up to: [batch, k] in float64."""
    scale = torch.exp2(exps.double()).repeat_interleave(32, dim=-1)
    return (digits.double() * 0.5 * scale).sum(0)


class Gemv:
    """One MXFP4 matrix on the tcgen05 path: out[m] = W x[m] for up to 8 sequences."""

    def __init__(self, packed, scales, device="cuda", splits=None, pieces=6, grid=0, spin_limit_ms=2000):
        if not torch.cuda.is_available():
            raise RuntimeError("the tcgen05 GEMV needs a CUDA device; there is no CPU path")
        self.rows, self.k = packed.shape[0], packed.shape[1] * 2
        if splits is None:
            splits = 1
            while self.k // splits > MAX_SLICE_K or self.k % (splits * CHUNK_K):
                splits += 1
                if splits > MAX_SPLITS:
                    raise ValueError(f"k = {self.k} does not split into at most {MAX_SPLITS} slices of whole chunks")
        self.splits, self.pieces, self.grid = splits, pieces, grid
        self.device = torch.device(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.w = pack(packed.to(self.device), scales.to(self.device), splits)
        self.lib = lib()
        nbytes = self.lib.mk_umma_scratch_bytes(self.rows, self.k, 8, splits, self.device.index, grid)
        if nbytes < 0:
            _lib.check(int(nbytes))
        self.part = torch.empty(max(nbytes, 16) // 4, dtype=torch.float32, device=self.device)
        self.cnt = torch.zeros((self.rows + ROWS - 1) // ROWS, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.spin_limit_ns = int(spin_limit_ms * 1e6)

    @property
    def weight_bytes(self):
        return self.w.numel()

    def __call__(self, x, out=None, round_bf16=True, stream=None, prof=None):
        """x fp32 [batch, k] on the device -> fp32 [batch, rows].  The launch is asynchronous; `check()` reads the status."""
        if x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] != self.k or not x.is_contiguous():
            raise ValueError(f"x: contiguous fp32 [batch, {self.k}]")
        batch = x.shape[0]
        if out is None:
            out = torch.empty(batch, self.rows, dtype=torch.float32, device=self.device)
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        a = UmmaArgs(w=self.w.data_ptr(), x=x.data_ptr(), out=out.data_ptr(), part=self.part.data_ptr(), cnt=self.cnt.data_ptr(),
                     status=self.status.data_ptr(), stream=s.cuda_stream, prof=prof.data_ptr() if prof is not None else 0, spin_limit_ns=self.spin_limit_ns, rows=self.rows,
                     k=self.k, batch=batch, pieces=self.pieces, splits=self.splits, device=self.device.index,
                     round_bf16=int(round_bf16), grid=self.grid)
        _lib.check(self.lib.mk_umma_gemv(ctypes.byref(a)))
        return out

    def check(self):
        st = self.status.cpu().tolist()
        if st[0]:
            self.status.zero_()
            self.cnt.zero_()
            raise RuntimeError(f"tcgen05 GEMV: wait {st[0]} ran out in CTA {st[1]} (detail {st[2]})")


def measure(rows, k, batch, pieces=6, splits=None, reps=20, seed=0, copies=0):
    """GB/s of packed weight bytes through the kernel: CUDA events around `reps` launches that walk over `copies`
    separately packed matrices (0 = as many as exceed the L2 four times), so no launch finds its weights in L2."""
    from . import quant as Q
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(seed)
    w = torch.randn(rows, k, generator=g, device=dev) * 0.02
    packed, scales = Q.quantize_mxfp4(w)
    op = Gemv(packed, scales, device=dev, splits=splits, pieces=pieces)
    if copies <= 0:
        copies = max(2, -(-4 * 126 * 2 ** 20 // op.weight_bytes))
    mats = [op.w] + [op.w.clone() for _ in range(copies - 1)]
    x = torch.randn(batch, k, generator=g, device=dev)
    out = torch.empty(batch, rows, dtype=torch.float32, device=dev)
    for i in range(3):
        op.w = mats[i % copies]
        op(x, out)
    torch.cuda.synchronize()
    op.check()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        op.w = mats[i % copies]
        op(x, out)
    e1.record()
    torch.cuda.synchronize()
    op.check()
    us = e0.elapsed_time(e1) * 1e3 / reps
    # one more launch with time stamps: per phase, the median over the CTAs that had work
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    stamps = torch.zeros(sms, 8, dtype=torch.int64, device=dev)
    op.w = mats[reps % copies]
    op(x, out, prof=stamps)
    torch.cuda.synchronize()
    t = stamps.cpu().double()
    t = t[t[:, 4] > 0]
    first = float(t[:, 0].min())
    ph = {"start_spread": float(t[:, 0].max()) - first, "planes_staged": float((t[:, 1] - t[:, 0]).median()),
          "first_chunk": float((t[:, 2] - t[:, 1]).median()), "stream": float((t[:, 3] - t[:, 2]).median()),
          "last_accumulator": float((t[:, 4] - t[:, 3]).median()), "epilogue": float((t[:, 5] - t[:, 4]).median()),
          "whole": float(t[:, 5].max()) - first}
    return {"phases_us": {k: round(v / 1e3, 2) for k, v in ph.items()},"rows": rows, "k": k, "batch": batch, "pieces": pieces, "splits": op.splits, "us_per_launch": us,
            "weight_bytes": op.weight_bytes, "gbs": op.weight_bytes / us / 1e3, "copies": copies}


def main(argv=None):
    import argparse
    import json
    ap = argparse.ArgumentParser(description="time the tcgen05 MXFP4 GEMV on the 27B model's projections")
    ap.add_argument("--shape", action="append", default=None, help="rows,k (default: the 27B gate/up and down projections)")
    ap.add_argument("--batch", type=int, action="append", default=None)
    ap.add_argument("--pieces", type=int, default=6)
    ap.add_argument("--splits", type=int, default=0, help="K slices (0: as few as fit)")
    ap.add_argument("--reps", type=int, default=20)
    a = ap.parse_args(argv)
    shapes = [tuple(int(v) for v in s.split(",")) for s in (a.shape or ["34816,5120", "5120,17408"])]
    for rows, k in shapes:
        for batch in a.batch or [1, 8]:
            print(json.dumps(measure(rows, k, batch, pieces=a.pieces, splits=a.splits or None, reps=a.reps)), flush=True)


if __name__ == "__main__":
    main()
