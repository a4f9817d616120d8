"""ctypes mirror of `include/mk_stage.h`.

The enumerators are read from the header itself, so the field indices the Python program builder uses
cannot drift from the ones the kernel was compiled with.  The structs mirror `mk_stage_desc` and
`mk_stage_args` field for field (the ABI test checks sizes and offsets against the C compiler).
"""

import ctypes
import os
import re

from .. import _lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "include", "mk_stage.h")


def _parse_enums(path):
    with open(path) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    names = {}
    for body in re.findall(r"enum\s*\{(.*?)\}", text, flags=re.S):
        value = -1
        for item in body.split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, expr = [x.strip() for x in item.split("=", 1)]
                value = int(eval(expr, {}, dict(names)))
            else:
                name, value = item, value + 1
            names[name] = value
    for name, expr in re.findall(r"#define\s+(MKS_\w+)\s+(\d+)", text):
        names[name] = int(expr)
    return names


K = _parse_enums(HEADER)
globals().update(K)          # MKS_OP_GEMV, MKS_I_TILES, ... as module attributes

I_COUNT, F_COUNT, P_COUNT = K["MKS_I_COUNT"], K["MKS_F_COUNT"], K["MKS_P_COUNT"]
MAX_BATCH, MAX_RANKS = K["MKS_MAX_BATCH"], K["MKS_MAX_RANKS"]


class StageDesc(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int32), ("flags", ctypes.c_int32), ("i", ctypes.c_int32 * I_COUNT),
                ("f", ctypes.c_float * F_COUNT), ("p", ctypes.c_uint64 * P_COUNT)]


class StageArgs(ctypes.Structure):
    _fields_ = [("program", ctypes.c_uint64), ("n_stages", ctypes.c_int32), ("batch", ctypes.c_int32),
                ("n_steps", ctypes.c_int32), ("device", ctypes.c_int32), ("tok", ctypes.c_uint64), ("pos", ctypes.c_uint64),
                ("tokens_out", ctypes.c_uint64), ("barrier", ctypes.c_uint64), ("barrier_base", ctypes.c_uint64),
                ("status", ctypes.c_uint64), ("spin_limit_ns", ctypes.c_int64), ("prof", ctypes.c_uint64),
                ("tp", ctypes.c_int32), ("rank", ctypes.c_int32), ("mailbox", ctypes.c_uint64 * MAX_RANKS),
                ("ar_base", ctypes.c_uint64), ("grid", ctypes.c_int32), ("prof_cta", ctypes.c_int32),
                ("tokens_in", ctypes.c_uint64), ("xs_bytes", ctypes.c_int32), ("n_tokens_in", ctypes.c_int32),
                ("row_valid", ctypes.c_uint64)]


STAGE_EXPORTS = ["mk_stage_launch", "mk_stage_validate", "mk_stage_count", "mk_stage_query", "mk_stage_scratch_bytes", "mk_sync_probe", "mk_peer_alloc", "mk_peer_open",
                 "mk_peer_close", "mk_peer_free"]
STAGE_QUERIES = ["SMEM_BYTES", "N_THREADS", "SLOT_BYTES", "XS_BYTES", "DESC_BYTES", "MAX_GROUPS", "MAILBOX_BYTES", "ATTN_MAX_CHUNK"]

_bound = False


def lib():
    """The shared library with the stage entry points bound."""
    global _bound
    L = _lib.load()
    if not _bound:
        P = ctypes.POINTER
        L.mk_stage_launch.argtypes = [P(StageArgs), ctypes.c_void_p]
        L.mk_stage_validate.argtypes = [P(StageDesc), ctypes.c_int, ctypes.c_int]
        L.mk_stage_count.argtypes = [P(StageDesc), ctypes.c_int, P(ctypes.c_int64), P(ctypes.c_int64)]
        L.mk_stage_query.argtypes = [ctypes.c_int]
        L.mk_stage_query.restype = ctypes.c_int64
        L.mk_stage_scratch_bytes.argtypes = [P(StageDesc), ctypes.c_int, ctypes.c_int]
        L.mk_stage_scratch_bytes.restype = ctypes.c_int64
        L.mk_sync_probe.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, P(ctypes.c_int64)]
        L.mk_peer_alloc.argtypes = [ctypes.c_int, ctypes.c_int64, P(ctypes.c_uint64), P(ctypes.c_uint8)]
        L.mk_peer_open.argtypes = [ctypes.c_int, P(ctypes.c_uint8), P(ctypes.c_uint64)]
        L.mk_peer_close.argtypes = [ctypes.c_uint64]
        L.mk_peer_free.argtypes = [ctypes.c_uint64]
        for name in STAGE_EXPORTS:
            if name not in ("mk_stage_query", "mk_stage_scratch_bytes"):
                getattr(L, name).restype = ctypes.c_int
        _bound = True
    return L


def query(name):
    return int(lib().mk_stage_query(STAGE_QUERIES.index(name)))


def desc(op, flags=0, i=None, f=None, p=None):
    """A stage record from {field name or index: value} dicts (names without the MKS_I_/F_/P_ prefix)."""
    d = StageDesc()
    d.op, d.flags = op, flags
    for prefix, arr, vals, conv in (("MKS_I_", d.i, i, int), ("MKS_F_", d.f, f, float), ("MKS_P_", d.p, p, int)):
        for key, v in (vals or {}).items():
            arr[K[prefix + key] if isinstance(key, str) else key] = conv(v)
    return d
