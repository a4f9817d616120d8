"""Cost of the stage-machine kernel's grid barrier, measured with the kernel itself.

`barrier_us(n)` launches a program of one (16-element) embedding stage followed by `n` empty stages, each
closed by a grid barrier, and returns microseconds per barrier from CUDA events.  The counterpart of the
reference's barrier microbenchmark (`qwen3.5-0.8b/bench/barrier.cu:27-59`): the number that says how much of a
decode step is synchronisation (stages per step x this).
"""

import torch

from . import desc as D
from .runtime import Program, Runtime


def barrier_us(n_barriers=2000, device="cuda", reps=5):
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    grid = torch.cuda.get_device_properties(dev).multi_processor_count
    pr = Program(dev, 1, grid)
    table = pr.zeros(1, 16, dtype=torch.bfloat16)
    h, ssq = pr.zeros(1, 16), pr.zeros(1, 1)
    pr.embed(table, h, ssq, None, 16, 1, keys_valid=False)
    for _ in range(n_barriers):
        pr.add(D.desc(D.MKS_OP_VEC, i=dict(VEC_N=0)))
    rt = Runtime(pr)
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rt.launch(1)
        e1.record()
        torch.cuda.synchronize()
        rt.check()
        best = min(best, e0.elapsed_time(e1) * 1e3 / (n_barriers + 1))
    return best


def sync_ns(mode, iters=2000, stores=0, device=0):
    """`mk_sync_probe`: 'barrier' = the bare grid-barrier protocol over one CTA per SM, 'hop' = a flag round trip
    between two CTAs; nanoseconds per iteration."""
    import ctypes
    from .. import _lib
    out = ctypes.c_int64()
    _lib.check(D.lib().mk_sync_probe(device, {"barrier": 0, "hop": 1}[mode], iters, stores, ctypes.byref(out)))
    return out.value


if __name__ == "__main__":
    for n in (200, 2000):
        print(f"stage kernel, {n} empty stages: {barrier_us(n):.3f} us per stage barrier")
    for stores in (0, 1, 4):
        print(f"bare grid barrier, {stores} store(s) per thread before it: {sync_ns('barrier', stores=stores)} ns")
    print(f"flag round trip between two CTAs: {sync_ns('hop')} ns")
