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
        pr.add(D.desc(D.MKS_OP_VEC))
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


if __name__ == "__main__":
    for n in (200, 2000):
        print(f"{n} barriers: {barrier_us(n):.3f} us per barrier")
