"""include/mk_umma.h against the built library and its ctypes mirror; the packed weight layout; the input digit
planes (no GPU: shape refusals and the scratch size make no CUDA call when the grid is given)."""

import ctypes
import os
import re
import shutil
import subprocess

import pytest
import torch

from megakernels_b200 import _lib
from megakernels_b200.stage import quant as Q
from megakernels_b200.stage import umma as U


def header_text():
    with open(U.HEADER) as f:
        return re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)


def test_every_declared_function_is_exported(lib_built):
    lib = ctypes.CDLL(lib_built)
    declared = set(re.findall(r"\b(mk_[a-z0-9_]+)\s*\(", header_text()))
    assert declared == set(U.UMMA_EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_layout_and_constants_match_the_c_compiler(lib_built, tmp_path):
    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    fields = [f for f, _ in U.UmmaArgs._fields_]
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "mk_umma.h"\nint main(void) {\n'
                   '  printf("%zu %d %d %d %d %d ", sizeof(mk_umma_args), MKU_ROWS, MKU_CHUNK_K, MKU_CHUNK_BYTES, MKU_MAX_SLICE_K, MKU_MAX_SPLITS);\n'
                   + "".join(f'  printf("%zu ", offsetof(mk_umma_args, {f}));\n' for f in fields) + '  return 0; }\n')
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.dirname(U.HEADER), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [ctypes.sizeof(U.UmmaArgs), U.ROWS, U.CHUNK_K, U.CHUNK_BYTES, U.MAX_SLICE_K, U.MAX_SPLITS]
    want += [getattr(U.UmmaArgs, f).offset for f in fields]
    assert got == want


def test_packed_chunks_hold_every_value_where_the_header_says(lib_built):
    g = torch.Generator().manual_seed(3)
    rows, k, splits = 200, 512, 2
    w = torch.randn(rows, k, generator=g) * 0.05
    packed, scales = Q.quantize_mxfp4(w)
    codes = Q.mxfp4_codes(packed)
    chunks = U.pack(packed, scales, splits)
    cps = k // splits // U.CHUNK_K
    assert chunks.shape == (splits, 2, cps, U.CHUNK_BYTES) and chunks.dtype == torch.uint8
    for r, c in ((0, 0), (7, 31), (8, 32), (127, 255), (128, 256), (199, 511), (37, 300)):
        s, kc = divmod(c // U.CHUNK_K, cps)
        ch = chunks[s, r // 128, kc]
        rr, cc = r % 128, c % 128
        byte = ch[(rr // 8) * 512 + (cc // 32) * 128 + (rr % 8) * 16 + (cc % 32) // 2]
        assert int((byte >> (4 * (cc & 1))) & 15) == int(codes[r, c]), (r, c)
        assert int(ch[8192 + (rr % 32) * 16 + (rr // 32) * 4 + cc // 32]) == int(scales[r, c // 32]), (r, c)
    # the padding rows are zero values with unit scales
    assert int(chunks[:, 1, :, :8192].reshape(splits, cps, 16, 4, 8, 16)[:, :, 9:].max()) == 0
    with pytest.raises(ValueError):
        U.pack(packed, scales, 3)


@pytest.mark.parametrize("rows,k,splits", [(128, 128, 1), (200, 512, 2), (1000, 1024, 4), (384, 2176 * 2, 2)])
def test_unpacking_the_chunks_gives_back_every_byte(rows, k, splits):
    g = torch.Generator().manual_seed(rows + k)
    packed, scales = Q.quantize_mxfp4(torch.randn(rows, k, generator=g) * 0.1)
    back_p, back_s = U.unpack(U.pack(packed, scales, splits), rows)
    assert torch.equal(back_p, packed) and torch.equal(back_s, scales)


@pytest.mark.parametrize("pieces", [4, 6, 8])
def test_digit_planes_restore_the_bf16_inputs(pieces):
    g = torch.Generator().manual_seed(pieces)
    x = torch.randn(3, 256, generator=g) * torch.logspace(-3, 2, 256)[None]      # a wide range inside the blocks
    x[1, 32:64] = 0.0                                                            # an all-zero block
    x[2, 5] = 0.0
    digits, exps = U.digit_planes(x, pieces)
    assert int(digits.abs().max()) <= 3
    want = x.to(torch.bfloat16).double()
    got = U.planes_value(digits, exps)
    blockmax = want.reshape(3, 8, 32).abs().amax(-1).repeat_interleave(32, dim=-1)
    # half a unit of the least significant digit: 2^(e + 1 - 2P) / 2 with 2^e <= blockmax
    assert bool(((got - want).abs() <= blockmax * 2.0 ** (-2 * pieces) + 1e-300).all())
    # the largest value of every block is exact (bf16 has 8 significant bits, 2 * pieces >= 8)
    big = want.abs() == blockmax
    assert torch.equal(got[big], want[big])


def test_shapes_the_kernel_cannot_hold_are_refused_before_any_cuda_call(lib_built):
    L = U.lib()
    ok = dict(w=256, x=256, out=256, cnt=256, status=256, rows=256, k=512, batch=2, pieces=6, splits=1, device=0, grid=8)
    for bad, text in ((dict(batch=9), b"batch"), (dict(k=500), b"columns per split"), (dict(k=8192), b"columns per split"),
                      (dict(splits=9), b"splits"), (dict(pieces=3), b"digit planes"), (dict(w=0), b"missing"), (dict(x=260), b"aligned"),
                      (dict(rows=0), b"rows"), (dict(splits=2, grid=1), b"CTAs")):
        a = U.UmmaArgs(**{**ok, **bad})
        assert L.mk_umma_gemv(ctypes.byref(a)) == _lib.MK_ERR_BADARG, bad
        assert text in L.mk_last_error(), (bad, L.mk_last_error())
    assert L.mk_umma_gemv(None) == _lib.MK_ERR_BADARG
    # 272 row blocks of 40 chunks on 148 CTAs: no row block is shared by more than three CTAs
    n = L.mk_umma_scratch_bytes(34816, 5120, 8, 1, 0, 148)
    assert n > 0 and n % (272 * 8 * 128 * 4) == 0 and n // (272 * 8 * 128 * 4) in (2, 3)
    assert L.mk_umma_scratch_bytes(34816, 5000, 8, 1, 0, 148) == _lib.MK_ERR_BADARG
