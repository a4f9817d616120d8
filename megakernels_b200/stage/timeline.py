"""Per-stage timeline of one decode step of the stage-machine kernel, from the kernel's own timestamps.

`Runtime.launch(prof=buffer)` makes consumer thread 0 of one CTA (or of every CTA with `prof_cta=-1`) record, for
each stage of the launch's last step, GPU-nanosecond stamps: stage entered, input staged (GEMV), work done,
barrier passed.  `profile(engine)` runs two steps, stamps the second and returns one row per stage name:
how many stages carry the name, the mean time from entering to the input being staged, to the work being done,
the wait at the barrier (imbalance between CTAs plus the barrier itself), and the name's share of the step.
The counterpart of the reference's timeline tool (`qwen3.5-0.8b/tools/timeline.py:49-97`); a profiler sees the
megakernel as one opaque kernel.
"""

import torch


def profile(engine, cta=0):
    """engine: any of the stage-machine engines (has `.rt`, `.M`).  Returns (rows, step microseconds)."""
    rt = engine.rt
    prof = torch.zeros(rt.n_stages, 8, dtype=torch.int64, device=rt.device)
    tok = rt.tok[: engine.M].clone()
    rt.launch(2, prof=prof, prof_cta=cta)
    torch.cuda.synchronize(rt.device)
    rt.check()
    rt.tok[: engine.M].copy_(tok)
    p = prof.cpu().double() / 1e3
    names = rt.prog.names
    rows, order = {}, []
    for i, name in enumerate(names):
        r = p[i]
        enter, staged, done, out = float(r[0]), float(r[1]), float(r[2]), float(r[3])
        if name not in rows:
            rows[name] = dict(name=name, n=0, stage_x=0.0, work=0.0, barrier=0.0, total=0.0)
            order.append(name)
        a = rows[name]
        a["n"] += 1
        a["stage_x"] += staged - enter if staged > 0 else 0.0
        a["work"] += done - (staged if staged > 0 else enter)
        a["barrier"] += out - done
        a["total"] += out - enter
    step_us = float(p[-1][3] - p[0][0])
    return [rows[n] for n in order], step_us


def format_rows(rows, step_us):
    lines = ["| stage | count | input staged µs | work µs | barrier wait µs | total µs each | µs per step | share |", "|---|---|---|---|---|---|---|---|"]
    for a in rows:
        n = a["n"]
        lines.append(f"| {a['name']} | {n} | {a['stage_x'] / n:.2f} | {a['work'] / n:.2f} | {a['barrier'] / n:.2f} | {a['total'] / n:.2f} | "
                     f"{a['total']:.0f} | {100 * a['total'] / step_us:.1f} % |")
    lines.append(f"| step | | | | | | {step_us:.0f} | |")
    return "\n".join(lines)


def main():
    import argparse
    ap = argparse.ArgumentParser(description="Per-stage timeline of a decode step (synthetic weights).")
    ap.add_argument("--model", default="qwen27b", choices=["qwen27b", "qwen35moe", "gemma26b"])
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=2048)
    args = ap.parse_args()
    import importlib
    pkg = importlib.import_module(f"megakernels_b200.{args.model}")
    shape = pkg.FULL.with_(layers=args.layers)
    kw = dict(keep_dequant=False) if args.model == "qwen27b" else (dict(keep_dense=False) if args.model == "qwen35moe" else {})
    W = pkg.SynthWeights(shape, layers=args.layers, device="cuda", draw_device="cuda", **kw)
    PK = pkg.Packed(W, "cuda")
    del W
    torch.cuda.empty_cache()
    eng = pkg.Engine(PK, args.batch, maxlen=args.context + 64)
    # a context of `context` positions: cached keys and values of any content cost the same to read
    for name in ("k_cache", "v_cache", "ks", "vs", "kf", "vf"):
        if hasattr(eng, name):
            getattr(eng, name).normal_()
    eng.rt.pos[: args.batch] = args.context
    eng.generate(torch.zeros(args.batch, dtype=torch.int32, device="cuda"), 4)
    rows, step_us = profile(eng)
    print(f"{args.model}, {args.layers} layers, batch {args.batch}, context {args.context}: {step_us:.0f} us per step (CTA 0's clock)\n")
    print(format_rows(rows, step_us))


if __name__ == "__main__":
    main()
