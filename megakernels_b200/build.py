"""Build the CUDA library in-tree for sm_100a with nvcc (no JIT cache, no torch extension).

`python -m megakernels_b200.build` compiles `csrc/mk_api.cu` into `libmk_b200.so` next to this
file.  The reference JIT-compiles its extension at import time instead
(`qwen3.5-0.8b/qwen_mk/_ext.py:12-30`); here the library is prebuilt so that it can be carried to
a machine and loaded without a compiler.  `MK_B200_DEFINES` adds `-D...` flags for A/B builds, the
counterpart of the reference's `QWEN_MK_DEFINES`.
"""

import os
import shlex
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, os.environ.get("MK_B200_LIBNAME", "libmk_b200.so"))
SOURCES = ["mk_api.cu", "mk_stage_api.cu", "mk_umma.cu"]
HEADERS = ["mk_common.h", "mk_device.cuh", "mk_decode.cuh", "mk_batch.cuh", "mk_stage.cuh", "mk_stage_ops.cuh",
           os.path.join("..", "..", "include", "mk_b200.h"), os.path.join("..", "..", "include", "mk_stage.h"),
           os.path.join("..", "..", "include", "mk_umma.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--fmad=false",
              "-Xcompiler", "-fPIC"]


def stale(lib=None):
    LIB = lib if lib is not None else globals()["LIB"]
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    csrc = os.path.join(HERE, "csrc")
    return any(os.path.getmtime(os.path.join(csrc, f)) > t for f in SOURCES + HEADERS)


CHAOS_LIB = os.path.join(HERE, "libmk_b200_chaos.so")


def build(force=False, verbose=False, lib=None, defines=None):
    """Compile if the library is missing or older than its sources.  Returns the library path.  `lib` / `defines`
    override the output file and the extra -D flags (default: MK_B200_LIBNAME / MK_B200_DEFINES)."""
    LIB = lib if lib is not None else globals()["LIB"]
    if not force and not stale(LIB):
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    csrc = os.path.join(HERE, "csrc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    defines = shlex.split(os.environ.get("MK_B200_DEFINES", "")) if defines is None else list(defines)
    # one object per translation unit, compiled side by side, then one link
    jobs = []
    for src in SOURCES:
        obj = os.path.join(objdir, os.path.basename(LIB) + "." + src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *defines, "-c", "-o", obj, os.path.join(csrc, src)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
            print(" ".join(cmd))
        jobs.append((obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = ""
    failed = False
    for obj, proc in jobs:
        text, _ = proc.communicate()
        log += text
        failed |= proc.returncode != 0
    if verbose:
        print(log)
    if failed:
        raise RuntimeError("nvcc failed:\n" + log)
    link = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *[o for o, _ in jobs]],
                          capture_output=True, text=True)
    if link.returncode != 0:
        raise RuntimeError("link failed:\n" + link.stdout + link.stderr)
    return LIB


def build_chaos(force=False):
    """The race-detection build (-DMK_CHAOS: pseudo-random pauses before publishes), beside the normal library."""
    return build(force=force, lib=CHAOS_LIB, defines=["-DMK_CHAOS"])


if __name__ == "__main__":
    if "--chaos" in sys.argv:
        print(build_chaos(force="--force" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
