"""include/mk_stage.h against the built library and the ctypes mirror; program validation (no GPU needed:
`mk_stage_validate`, `mk_stage_count`, `mk_stage_scratch_bytes` and `mk_stage_query` make no CUDA call)."""

import ctypes
import os
import re
import shutil
import subprocess

import pytest

from megakernels_b200 import _lib
from megakernels_b200.stage import desc as D
from megakernels_b200.stage import pack as P

HEADER = D.HEADER


def header_text():
    with open(HEADER) as f:
        return re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)


def test_every_declared_function_is_exported(lib_built):
    lib = ctypes.CDLL(lib_built)
    declared = set(re.findall(r"\b(mk_[a-z0-9_]+)\s*\(", header_text()))
    assert declared == set(D.STAGE_EXPORTS)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in mk_stage.h but not exported"


def test_queries_follow_the_header_order(lib_built):
    names = [n for n in D.K if n.startswith("MKS_Q_")]
    assert [n[len("MKS_Q_"):] for n in sorted(names, key=D.K.get)] == D.STAGE_QUERIES
    assert D.query("DESC_BYTES") == ctypes.sizeof(D.StageDesc) == 288
    assert D.query("SMEM_BYTES") <= 227 * 1024
    assert D.query("N_THREADS") == 544 and D.query("SLOT_BYTES") == P.SLOT_BYTES
    assert D.lib().mk_stage_query(999) == -1


def test_struct_layouts_match_the_c_compiler(lib_built, tmp_path):
    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    fields = ["program", "n_steps", "tok", "barrier_base", "spin_limit_ns", "tp", "mailbox", "ar_base", "grid", "tokens_in", "xs_bytes", "n_tokens_in", "row_valid"]
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "mk_stage.h"\nint main(void) {\n'
                   '  printf("%zu %zu %zu %zu %zu ", sizeof(mk_stage_desc), offsetof(mk_stage_desc, i), offsetof(mk_stage_desc, f), '
                   'offsetof(mk_stage_desc, p), sizeof(mk_stage_args));\n'
                   + "".join(f'  printf("%zu ", offsetof(mk_stage_args, {f}));\n' for f in fields)
                   + '  return 0; }\n')
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.dirname(HEADER), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [ctypes.sizeof(D.StageDesc), D.StageDesc.i.offset, D.StageDesc.f.offset, D.StageDesc.p.offset, ctypes.sizeof(D.StageArgs)]
    want += [getattr(D.StageArgs, f).offset for f in fields]
    assert got == want


def test_field_counts_leave_room_for_every_index():
    for prefix, count in (("MKS_I_", D.I_COUNT), ("MKS_F_", D.F_COUNT), ("MKS_P_", D.P_COUNT)):
        used = [v for k, v in D.K.items() if k.startswith(prefix) and not k.endswith("_COUNT")]
        assert used and max(used) < count, prefix


def _gemv(**over):
    i = dict(FMT=D.MKS_FMT_BF16, TILES=8, SPLITS=1, GROUPS=1, UNIT_STEPS=16, CHUNK_STEPS=8, CHUNK_BYTES=4096, KC=256,
             PROLOGUE=D.MKS_P_PLAIN, EPILOGUE=D.MKS_E_STORE, N_VALID=128, X_STRIDE=256, OUT_STRIDE=128, K_TOTAL=256, PIECES=1)
    p = dict(W=0x1000, X=0x2000, OUT=0x3000, W_BYTES=8 * 16 * 512)
    for k, v in over.items():
        (p if k in ("W", "X", "OUT", "CNT", "PART", "KEYS", "X_SSQ", "NORM_W") else i)[k] = v
    return D.desc(D.MKS_OP_GEMV, 0, i=i, p=p)


def _embed():
    return D.desc(D.MKS_OP_EMBED, 0, i=dict(HIDDEN=256, VOCAB=100), p=dict(TABLE=0x100, H=0x200, H_SSQ=0x300))


def _validate(stages, batch=2):
    arr = (D.StageDesc * len(stages))(*stages)
    return D.lib().mk_stage_validate(arr, len(stages), batch)


def test_a_well_formed_program_validates(lib_built):
    assert _validate([_embed(), _gemv()]) == _lib.MK_OK
    nb, na = ctypes.c_int64(), ctypes.c_int64()
    prog = [_embed(), _gemv(), _gemv(ALLREDUCE=1)]
    prog[1].flags = D.MKS_FLAG_NO_BARRIER
    arr = (D.StageDesc * 3)(*prog)
    assert D.lib().mk_stage_count(arr, 3, ctypes.byref(nb), ctypes.byref(na)) == _lib.MK_OK
    assert (nb.value, na.value) == (2, 1)
    # staging: 8 sequences x (2 bytes x 256 columns rounded to 128, + 32) -> fits the minimum of 4096
    assert D.lib().mk_stage_scratch_bytes(arr, 3, 8) == max(4096, (512 + 32) * 8 + 127) // 128 * 128


@pytest.mark.parametrize("over,text", [
    (dict(FMT=9), b"weight format"),
    (dict(KC=64, UNIT_STEPS=4), b"fewer than 128"),
    (dict(UNIT_STEPS=15), b"unit steps"),
    (dict(CHUNK_STEPS=3), b"chunk steps"),
    (dict(CHUNK_BYTES=8192), b"chunk of"),
    (dict(CHUNK_BYTES=4100), b"chunk of"),
    (dict(SPLITS=2), b"counters"),
    (dict(W=0x1008), b"misaligned"),
    (dict(X=0), b"missing"),
    (dict(PROLOGUE=1), b"norm prologue"),
    (dict(EPILOGUE=3), b"key buffer"),
    (dict(PIECES=3), b"pieces"),
    (dict(GROUPS=0), b"groups"),
    (dict(KC=32768, UNIT_STEPS=2048), b"staging area"),
    (dict(TILES=0), b"tiles"),
])
def test_malformed_gemv_stages_are_refused(lib_built, over, text):
    assert D.MKS_P_NORM == 1 and D.MKS_E_LOGITS == 3
    assert _validate([_embed(), _gemv(**over)]) == _lib.MK_ERR_BADARG
    assert text in D.lib().mk_last_error(), D.lib().mk_last_error()


def test_program_level_refusals(lib_built):
    L = D.lib()
    assert L.mk_stage_validate(None, 0, 1) == _lib.MK_ERR_BADARG
    assert _validate([_gemv()]) == _lib.MK_ERR_BADARG and b"first stage" in L.mk_last_error()
    assert _validate([_embed()], batch=9) == _lib.MK_ERR_BADARG and b"batch" in L.mk_last_error()
    assert _validate([_embed(), D.desc(77)]) == _lib.MK_ERR_BADARG and b"unknown op" in L.mk_last_error()
    attn = dict(NQ=24, NKV=4, HD=256, CHUNK_POS=64, MAX_CHUNKS=16)
    assert _validate([_embed(), D.desc(D.MKS_OP_ATTN, i=attn)]) == _lib.MK_OK
    for bad, text in ((dict(HD=128), b"head dim"), (dict(CHUNK_POS=8), b"positions per task"), (dict(NQ=64), b"query heads"),
                      (dict(MAX_CHUNKS=1000), b"split records")):
        assert _validate([_embed(), D.desc(D.MKS_OP_ATTN, i={**attn, **bad})]) == _lib.MK_ERR_BADARG
        assert text in L.mk_last_error()
    assert _validate([_embed(), D.desc(D.MKS_OP_ROUTE, i=dict(EXPERTS=100, TOPK=8))]) == _lib.MK_ERR_BADARG
    assert _validate([_embed(), D.desc(D.MKS_OP_ROUTE, i=dict(EXPERTS=256, TOPK=8))], batch=8) == _lib.MK_OK
    assert _validate([_embed(), D.desc(D.MKS_OP_GDN, i=dict(NKH=16, NVH=40))]) == _lib.MK_ERR_BADARG


def test_launch_refuses_bad_arguments_before_touching_a_gpu(lib_built):
    L = D.lib()
    assert L.mk_stage_launch(None, None) == _lib.MK_ERR_BADARG
    ok = dict(program=0x1000, n_stages=1, batch=1, n_steps=1, device=0, tok=8, pos=16, barrier=64, status=128, tp=1, rank=0)
    for bad, text in ((dict(program=0), b"no program"), (dict(batch=9), b"batch"), (dict(n_steps=0), b"n_steps"),
                      (dict(tok=0), b"missing"), (dict(barrier=60), b"aligned"), (dict(tp=9), b"rank"), (dict(rank=1), b"rank"),
                      (dict(tp=2), b"mailbox")):
        a = D.StageArgs(**{**ok, **bad})
        assert L.mk_stage_launch(ctypes.byref(a), None) == _lib.MK_ERR_BADARG, bad
        assert text in L.mk_last_error(), (bad, L.mk_last_error())
