"""ctypes binding of `libmk_b200.so` (declarations: `include/mk_b200.h`).

There is no fallback: if the library is missing or a call fails, this raises.  The binding takes
the place of the reference's pybind module (`qwen3.5-0.8b/csrc/binding.cpp:107-121`); errors that
the reference raises through `TORCH_CHECK` / `C10_CUDA_CHECK` arrive as `MkError` (a
`RuntimeError`) carrying the library's message.
"""

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, os.environ.get("MK_B200_LIBNAME", "libmk_b200.so"))

MK_OK, MK_ERR_BADARG, MK_ERR_TIMEOUT, MK_ERR_CUDA, MK_ERR_UNSUPPORTED = 0, -1, -2, -3, -4
MK_QUANT = {"bf16": 0, "int8": 1}
MK_KV = {"bf16": 0, "fp32": 1}
MK_SHAPE_QWEN35_08B = 1

# index = value of the MK_L_* / MK_G_* / MK_Q_* enumerators in include/mk_b200.h
LAYER_FIELDS = ["w_in", "w_out", "w_gu", "w_down", "s_in", "s_out", "s_gu", "s_down", "in_norm", "post_norm",
                "conv_w", "A_log", "dt_bias", "gdn_norm", "conv_hist", "state", "state_bak", "q_norm", "k_norm",
                "k_cache", "v_cache", "kind", "conv_hist_b", "w_out_rows", "w_down_rows"]
GLOBAL_FIELDS = ["embed", "embed_scale", "lm_head", "lm_scale", "final_norm", "rope_cos", "rope_sin", "xl", "projl",
                 "mixl", "actl", "lml", "attn_part", "block_table", "status", "mtp_fc", "mtp_fc_scale",
                 "mtp_norm_e", "mtp_norm_h", "mtp_norm", "draft_head", "draft_scale", "draft_ids", "xml", "partl"]
QUERIES = ["SMEM_BYTES", "N_THREADS", "CONV_RING", "KV_BLOCK", "MAX_SPLITS", "PART_STRIDE", "OPS_PER_LAYER",
           "PROF_MAX_OPS", "PROF_FIELDS", "SPEC_T", "MAX_LAYERS", "LAYER_FIELDS", "GLOBAL_FIELDS", "SLOT_BYTES",
           "STAGES", "MAX_LM_ROWS", "MAX_BATCH", "BATCH_SMEM_BYTES"]
EXPORTS = ["mk_create", "mk_destroy", "mk_set_params", "mk_launch", "mk_launch_static", "mk_launch_batch", "mk_status", "mk_query", "mk_bw_probe",
           "mk_plan_rows", "mk_plan_attn_chunk", "mk_last_error"]


class MkError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"mk_b200 error {code}: {message}")
        self.code = code


class ModelDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("shape", "n_layers", "vocab", "max_seq", "quant", "kv_dtype", "draft_vocab", "device", "grid", "max_batch")]


class LaunchArgs(ctypes.Structure):
    _fields_ = [("forced", ctypes.c_uint64), ("n_forced", ctypes.c_int32), ("n_steps", ctypes.c_int32),
                ("lm_from", ctypes.c_int32), ("start_pos", ctypes.c_int32), ("epoch_base", ctypes.c_uint32),
                ("seed", ctypes.c_uint32), ("inv_temperature", ctypes.c_float), ("n_stop", ctypes.c_int32),
                ("stop_ids", ctypes.c_uint64), ("tokens_out", ctypes.c_uint64), ("logits_out", ctypes.c_uint64),
                ("resid_out", ctypes.c_uint64), ("step_ts", ctypes.c_uint64), ("out_info", ctypes.c_uint64),
                ("prof", ctypes.c_uint64), ("prof_step", ctypes.c_int32), ("grid", ctypes.c_int32),
                ("spin_limit_ns", ctypes.c_int64), ("spec", ctypes.c_int32),
                ("first_tok", ctypes.c_int32), ("first_draft", ctypes.c_int32), ("limit", ctypes.c_int32),
                ("spec_out", ctypes.c_uint64), ("cycle_out", ctypes.c_uint64)]


MAX_BATCH = 8


class BatchArgs(ctypes.Structure):
    _fields_ = [("forced", ctypes.c_uint64), ("n_forced", ctypes.c_int32 * MAX_BATCH),
                ("n_total", ctypes.c_int32 * MAX_BATCH), ("pos0", ctypes.c_int32 * MAX_BATCH),
                ("batch", ctypes.c_int32), ("n_steps", ctypes.c_int32), ("lm_from", ctypes.c_int32),
                ("epoch_base", ctypes.c_uint32), ("seed", ctypes.c_uint32), ("inv_temperature", ctypes.c_float),
                ("n_stop", ctypes.c_int32), ("prof_step", ctypes.c_int32), ("stop_ids", ctypes.c_uint64),
                ("tokens_out", ctypes.c_uint64), ("logits_out", ctypes.c_uint64), ("step_ts", ctypes.c_uint64),
                ("out_info", ctypes.c_uint64), ("prof", ctypes.c_uint64), ("spin_limit_ns", ctypes.c_int64)]


_lib = None


def load():
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise MkError(MK_ERR_UNSUPPORTED, f"{LIB_PATH} is missing: run `python -m megakernels_b200.build` "
                                           "(there is no CPU or PyTorch fallback for the decode kernel)")
    lib = ctypes.CDLL(LIB_PATH)
    P = ctypes.POINTER
    lib.mk_create.argtypes = [P(ModelDesc), P(ctypes.c_void_p)]
    lib.mk_destroy.argtypes = [ctypes.c_void_p]
    lib.mk_set_params.argtypes = [ctypes.c_void_p, P(ctypes.c_int64), ctypes.c_int64, P(ctypes.c_int64),
                                  ctypes.c_int64, P(ctypes.c_int64), ctypes.c_int64]
    lib.mk_launch.argtypes = [ctypes.c_void_p, P(LaunchArgs), ctypes.c_void_p]
    lib.mk_launch_static.argtypes = [ctypes.c_void_p, P(LaunchArgs), ctypes.c_void_p]
    lib.mk_launch_batch.argtypes = [ctypes.c_void_p, P(BatchArgs), ctypes.c_void_p]
    lib.mk_status.argtypes = [ctypes.c_void_p, P(ctypes.c_int32)]
    lib.mk_query.argtypes = [ctypes.c_int]
    lib.mk_query.restype = ctypes.c_int64
    lib.mk_bw_probe.argtypes = [ctypes.c_uint64, ctypes.c_int64, ctypes.c_int, ctypes.c_uint64, ctypes.c_int,
                                ctypes.c_void_p]
    lib.mk_plan_rows.argtypes = [ctypes.c_int] * 4 + [P(ctypes.c_int), P(ctypes.c_int)]
    lib.mk_plan_attn_chunk.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.mk_plan_attn_chunk.restype = ctypes.c_int
    lib.mk_last_error.restype = ctypes.c_char_p
    for name in ("mk_create", "mk_destroy", "mk_set_params", "mk_launch", "mk_launch_static", "mk_launch_batch", "mk_status", "mk_bw_probe", "mk_plan_rows"):
        getattr(lib, name).restype = ctypes.c_int
    _lib = lib
    return lib


def check(code):
    if code != MK_OK:
        raise MkError(code, load().mk_last_error().decode())


def query(name):
    return int(load().mk_query(QUERIES.index(name)))


def plan_rows(rows, unit, cta, grid):
    r0, r1 = ctypes.c_int(), ctypes.c_int()
    check(load().mk_plan_rows(rows, unit, cta, grid, ctypes.byref(r0), ctypes.byref(r1)))
    return r0.value, r1.value


def i64_array(values):
    return (ctypes.c_int64 * len(values))(*[int(v) for v in values])
