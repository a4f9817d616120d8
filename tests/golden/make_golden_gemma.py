"""Writes tests/golden/gemma26b_*.json from the reference's own exact-mode decoder of the 26B-A4B model.

Run where the reference checkout is present (it cannot travel to a GPU machine):

    python tests/golden/make_golden_gemma.py [reference root] [case name]

The reference decoder (`gemma4-26b-a4b-gfx942/mk/reference.py`, `step(..., mode="exact")`) fixes the model's widths
as module constants, so the fixtures are at the full widths (hidden 2816, 16 query heads, 8 x 256 sliding and
2 x 512 full KV heads, 128 experts of 704, dense MLP 2112) with the depth truncated to one pattern period
(5 sliding layers + 1 full) and the vocabulary cut to 4096 rows; the weights are the seeded synthetic ones of
`megakernels_b200.gemma26b.synth.SynthWeights` drawn on the CPU (FP8 e4m3 with one scale per output row).

Each fixture holds, per step: the greedy ids, soft-capped logits at fixed probe columns, the top-2 gap, the routed
expert ids of every layer and the distance between the 8th and the 9th router logit (a consumer whose arithmetic
differs in the last bits may choose differently where that distance is tiny, and is then on another trajectory).
"""

import json
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from megakernels_b200.gemma26b.dims import FULL  # noqa: E402
from megakernels_b200.gemma26b.synth import SynthWeights, make_prompt  # noqa: E402

CASES = [
    # name, layers, M, prompt length, generated steps, init, fmt, experts
    ("gemma26b_l6_m2_fp8", 6, 2, 4, 4, "realistic", "fp8", 128),
    # the CPU pin test replays this one: 16 experts instead of 128 keep its weights small (the decoder takes the
    # expert count from the router's rows)
    ("gemma26b_l6_m2_bf16", 6, 2, 3, 3, "realistic", "bf16", 16),
]
VOCAB = 4096
N_PROBE = 128


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference")
    only = sys.argv[2] if len(sys.argv) > 2 else None
    sys.path.insert(0, os.path.join(ref_root, "gemma4-26b-a4b-gfx942"))
    from mk import reference as R

    for name, layers, M, n_prompt, n_gen, init, fmt, experts in CASES:
        if only and name != only:
            continue
        t0 = time.time()
        shape = FULL.with_(vocab=VOCAB, layers=layers, experts=experts)
        W = SynthWeights(shape, layers=layers, seed=13, init=init, fmt=fmt, device="cpu")
        st = R.State.new(M, 64, device="cpu")
        prompts = [make_prompt(VOCAB, n_prompt, seed=j) for j in range(M)]
        gen = torch.Generator().manual_seed(99)
        probe = torch.randperm(VOCAB, generator=gen)[:N_PROBE].sort().values
        rec = {"name": name, "layers": layers, "M": M, "vocab": VOCAB, "seed": 13, "init": init, "fmt": fmt, "experts": experts,
               "prompts": prompts, "probe_indices": probe.tolist(), "steps": []}
        tok = None
        for t in range(n_prompt + n_gen):
            if t < n_prompt:
                tok = torch.tensor([p[t] for p in prompts])
            dump = {}
            logits = R.step(W, tok, st, layers=layers, dump=dump)
            top = logits.topk(2, dim=-1).values
            tok = logits.argmax(-1)
            rec["steps"].append({"ids": tok.tolist(), "probe_logits": logits[:, probe].tolist(),
                                 "top2_gap": (top[:, 0] - top[:, 1]).tolist(),
                                 "abs_sum": logits.double().abs().sum(-1).tolist(),
                                 "experts": [dump[i]["ids"].tolist() for i in range(layers)],
                                 "boundary_gap": [(lambda v: (v[:, 7] - v[:, 8]).tolist())(dump[i]["logits"].sort(-1, descending=True).values)
                                                  for i in range(layers)]})
        path = os.path.join(HERE, name + ".json")
        with open(path, "w") as f:
            json.dump(rec, f)
        print(f"{name}: {os.path.getsize(path) / 1e3:.0f} kB in {time.time() - t0:.0f} s", flush=True)


if __name__ == "__main__":
    main()
