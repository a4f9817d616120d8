"""Per-op timeline of one decode step from the kernel's own timestamps.

`Megakernel.run(prof=mk.prof_buffer(), prof_step=s)` makes consumer thread 0 of every CTA record, for
each op of step `s`, GPU-nanosecond stamps: op entered, inputs staged, work done (mixers), outputs
published, and the time spent waiting for ring chunks.  `summarize` turns the buffer into per-op-kind
figures: how long the median CTA waited for inputs and worked, and the critical path (last publish of
an op minus last publish of the op before).  The reference's `tools/timeline.py:49-97` reads its
kernel's stamp buffer the same way (ncu sees a megakernel as one opaque kernel).
"""

import numpy as np

OP_NAMES = ["in-proj", "mixer", "out-proj", "gate/up", "down"]


def summarize(prof, cfg):
    """prof: int64 tensor/array [grid, PROF_MAX_OPS, PROF_FIELDS].  Returns a list of dict rows."""
    p = np.asarray(prof.cpu() if hasattr(prof, "cpu") else prof).astype(np.int64)
    L = cfg.n_layers
    nops = 5 * L + 1
    p = p[:, :nops]
    enter, staged, pub, ringwait = p[..., 0], p[..., 1], p[..., 3], p[..., 4]
    last_pub = pub.max(0).astype(np.float64)
    crit = np.diff(last_pub, prepend=enter[:, 0].min())
    rows = []

    def add(label, sel):
        if not sel:
            return
        busy = pub[:, sel] - enter[:, sel]
        have = staged[:, sel] > 0
        wait = np.where(have, staged[:, sel] - enter[:, sel], 0)
        rows.append(dict(op=label, n=len(sel), wait_us=float(np.median(wait[have])) / 1e3 if have.any() else 0.0,
                         busy_us=float(np.median(busy)) / 1e3, busy_max_us=float(busy.max()) / 1e3,
                         ring_wait_us=float(np.median(ringwait[:, sel])) / 1e3,
                         critical_us=float(np.median(crit[sel])) / 1e3))

    for k, name in enumerate(OP_NAMES):
        for kind, tag in (("linear_attention", "deltanet"), ("full_attention", "attention")):
            add(f"{name} ({tag} layer)", [l * 5 + k for l in range(L) if cfg.layer_types[l] == kind])
    add("lm head", [5 * L])
    rows.append(dict(op="step", n=1, wait_us=0.0, busy_us=float(last_pub[-1] - enter[:, 0].min()) / 1e3,
                     busy_max_us=0.0, ring_wait_us=0.0, critical_us=float(crit.sum()) / 1e3))
    return rows


def format_rows(rows):
    out = [f"{'op':34s} {'n':>3s} {'wait':>7s} {'busy':>7s} {'busy max':>9s} {'ring wait':>9s} {'critical':>9s}  (us)"]
    for r in rows:
        out.append(f"{r['op']:34s} {r['n']:3d} {r['wait_us']:7.2f} {r['busy_us']:7.2f} {r['busy_max_us']:9.2f} "
                   f"{r['ring_wait_us']:9.2f} {r['critical_us']:9.2f}")
    return "\n".join(out)


def profile_step(mk, context_tokens, step=8, n_generate=16):
    """Feed `context_tokens`, generate, and return the summary rows of decode step `step`."""
    mk.reset()
    last = mk.prefill(context_tokens)
    prof = mk.prof_buffer()
    mk.run([last], n_generate=n_generate, prof=prof, prof_step=step)
    return summarize(prof, mk.cfg)


def main():
    import argparse

    from .config import qwen35_08b
    from .engine import Megakernel
    from .synth import make_prompt, make_weights
    ap = argparse.ArgumentParser(description="Per-op timeline of one decode step of the 0.8B kernels (synthetic weights, full size).")
    ap.add_argument("--quant", default="bf16", choices=["bf16", "int8"])
    ap.add_argument("--context", type=int, default=32)
    ap.add_argument("--batch", type=int, default=1)
    args = ap.parse_args()
    cfg = qwen35_08b()
    w = make_weights(cfg, 0)
    mk = Megakernel((cfg, w), max_seq=args.context + 64, quant=args.quant, batch=args.batch)
    if args.batch == 1:
        rows = profile_step(mk, make_prompt(cfg, args.context), step=8, n_generate=16)
    else:
        prompts = [make_prompt(cfg, args.context, seed=100 + j) for j in range(args.batch)]
        prof = mk.prof_buffer()
        mk.run_batch(prompts, n_generate=16, prof=prof, prof_step=args.context + 8)
        rows = summarize(prof, cfg)
    print(f"0.8B hybrid, {args.quant} weights, batch {args.batch}, context {args.context}: decode step 8 of a 16-step launch\n")
    print(format_rows(rows))
    print("\n(wait = entering an op until its inputs are staged; busy = entering until its outputs are published, median CTA;"
          "\n critical = last publish of the op minus last publish of the op before, median over the op's layers; the `step` row's"
          "\n critical column is the sum over all ops: the step's critical path)")


if __name__ == "__main__":
    main()
