"""The C-ABI library loads and exports what include/mk_b200.h declares (no compute: runs without a GPU)."""

import ctypes
import os
import re

import pytest

from megakernels_b200 import _lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "mk_b200.h")


def header_text():
    with open(HEADER) as f:
        return re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)


def enum_names(prefix):
    """Enumerators with the given prefix, in declaration order."""
    names = []
    for body in re.findall(r"enum\s*\{(.*?)\}", header_text(), flags=re.S):
        for item in body.split(","):
            name = item.split("=")[0].strip()
            if name.startswith(prefix):
                names.append(name)
    return names


def test_every_declared_function_is_exported(lib_built):
    lib = ctypes.CDLL(lib_built)
    declared = re.findall(r"\b(mk_[a-z0-9_]+)\s*\(", header_text())
    assert set(declared) == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in mk_b200.h but not exported"


def test_field_order_matches_header(lib_built):
    layer = [n for n in enum_names("MK_L_")]
    assert [n[len("MK_L_"):].lower() for n in layer] == [f.lower() for f in _lib.LAYER_FIELDS]
    glob = [n for n in enum_names("MK_G_")]
    assert [n[len("MK_G_"):].lower() for n in glob] == [f.lower() for f in _lib.GLOBAL_FIELDS]
    assert _lib.query("LAYER_FIELDS") == len(_lib.LAYER_FIELDS)
    assert _lib.query("GLOBAL_FIELDS") == len(_lib.GLOBAL_FIELDS)
    queries = enum_names("MK_Q_")
    assert [n[len("MK_Q_"):] for n in queries] == _lib.QUERIES


def test_struct_layouts(lib_built):
    assert ctypes.sizeof(_lib.ModelDesc) == 40
    a = _lib.LaunchArgs
    assert a.stop_ids.offset == 40 and a.prof_step.offset == 96 and a.spin_limit_ns.offset == 104
    assert a.spec.offset == 112 and a.spec_out.offset == 128 and ctypes.sizeof(a) == 144


def test_batch_args_layout_matches_the_header(lib_built, tmp_path):
    """The ctypes mirror of mk_batch_args has the size and offsets the C compiler gives the header's struct."""
    import shutil
    import subprocess
    b = _lib.BatchArgs
    assert ctypes.sizeof(b) == 192 and b.spin_limit_ns.offset == 184 and b.n_total.offset == 40 and b.batch.offset == 104 and b.stop_ids.offset == 136
    assert _lib.query("MAX_BATCH") == _lib.MAX_BATCH == 8
    assert _lib.query("BATCH_SMEM_BYTES") <= 227 * 1024
    if not shutil.which("gcc"):
        return
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "mk_b200.h"\n'
                   'int main(void) { printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(mk_batch_args), offsetof(mk_batch_args, n_total), '
                   'offsetof(mk_batch_args, batch), offsetof(mk_batch_args, stop_ids), sizeof(mk_launch_args), '
                   'sizeof(mk_model_desc)); return 0; }\n')
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.dirname(HEADER), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert got == [192, 40, 104, 136, ctypes.sizeof(_lib.LaunchArgs), ctypes.sizeof(_lib.ModelDesc)]


def test_constants(lib_built):
    assert _lib.query("N_THREADS") % 32 == 0
    assert _lib.query("SMEM_BYTES") <= 227 * 1024
    assert _lib.query("SLOT_BYTES") % 16 == 0
    assert _lib.query("KV_BLOCK") == 64 and _lib.query("CONV_RING") == 8
    assert _lib.load().mk_query(9999) == -1


def test_bad_arguments_are_refused_without_a_gpu(lib_built):
    lib = _lib.load()
    assert lib.mk_create(None, None) == _lib.MK_ERR_BADARG
    assert b"null" in lib.mk_last_error()
    desc = _lib.ModelDesc(shape=77, n_layers=4, vocab=4096, max_seq=64, quant=0, kv_dtype=1, draft_vocab=0, device=0, grid=0)
    h = ctypes.c_void_p()
    assert lib.mk_create(ctypes.byref(desc), ctypes.byref(h)) == _lib.MK_ERR_UNSUPPORTED
    with pytest.raises(_lib.MkError):
        _lib.check(lib.mk_plan_rows(10, 3, 0, 4, None, None))
    # per-sequence buffers: a batch capacity outside [0, 8], or more KV pages than one launch maps, is refused at creation
    for kw in (dict(max_batch=9), dict(max_batch=-1), dict(max_batch=8, max_seq=8192)):
        d = dict(shape=_lib.MK_SHAPE_QWEN35_08B, n_layers=4, vocab=4096, max_seq=64, quant=1, kv_dtype=1, draft_vocab=0,
                 device=0, grid=0, max_batch=0)
        d.update(kw)
        desc = _lib.ModelDesc(**d)
        assert lib.mk_create(ctypes.byref(desc), ctypes.byref(h)) == _lib.MK_ERR_BADARG, kw
        assert b"max_batch" in lib.mk_last_error() or b"KV pages" in lib.mk_last_error()
    assert lib.mk_launch(None, None, None) == _lib.MK_ERR_BADARG
    assert lib.mk_launch_batch(None, None, None) == _lib.MK_ERR_BADARG
    assert lib.mk_destroy(None) == _lib.MK_OK
