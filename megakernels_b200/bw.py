"""DRAM read bandwidth as the decode kernel can see it: the denominator check for roofline fractions.

Two kernels from the library stream a buffer once through every SM: plain 128-bit loads, and the
decode kernel's own bulk-copy ring (one producer lane, 6 x 32 KB stages, consumer warps reading
shared memory).  Same purpose as the reference's `common/bw.cu` (`read_vec`, `read_tma`), whose
measured number is the roofline its benchmarks quote (`qwen3.5-0.8b/README.md:115-116`).
"""

import ctypes

import torch

from . import _lib

MODES = {"plain": 0, "ring": 1}


def measure(mode="ring", gib=2.0, reps=5, device=None):
    """Best-of-`reps` read bandwidth in GB/s over a `gib` GiB buffer (larger than L2)."""
    lib = _lib.load()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    n = int(gib * (1 << 30)) // 32768 * 32768
    buf = torch.empty(n, dtype=torch.uint8, device=device)
    buf.random_(0, 255)
    sink = torch.zeros(4, dtype=torch.int32, device=device)
    stream = torch.cuda.current_stream(device)
    best = 0.0
    for _ in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        _lib.check(lib.mk_bw_probe(buf.data_ptr(), n, MODES[mode], sink.data_ptr(), device.index,
                                   ctypes.c_void_p(stream.cuda_stream)))
        e1.record(stream)
        e1.synchronize()
        best = max(best, n / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    return best


if __name__ == "__main__":
    for m in MODES:
        print(f"{m}: {measure(m):.0f} GB/s")
