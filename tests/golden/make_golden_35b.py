"""Writes tests/golden/qwen35moe_*.json from the reference's own exact-mode decoder of the 35B-A3B MoE model.

Run where the reference checkout is present (it cannot travel to a GPU machine):

    python tests/golden/make_golden_35b.py [reference root] [case name]

The reference decoder (`qwen3.6-35b-a3b-gfx942/mk/reference.py`, `step(..., emulate=False)`) fixes the model's
widths as module constants, so the fixtures are at the full widths (hidden 2048, 256 experts of intermediate 512,
top 8, 16/32 DeltaNet heads, 16/2 attention heads) with the depth truncated to one pattern period and the
vocabulary cut to 4096 rows; the weights are the seeded synthetic ones of
`megakernels_b200.qwen35moe.synth.SynthWeights` drawn on the CPU, FP8 e4m3 with 128 x 128 block scales,
dequantised exactly for the decoder as the reference does with the checkpoint (`reference.py:55-58`).

Each fixture holds, per step: the greedy ids, logits at fixed probe columns, the top-2 gap, the routed expert ids
and weights of every layer; after the last step sums over the recurrent state.
"""

import json
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from megakernels_b200.qwen35moe.dims import FULL  # noqa: E402
from megakernels_b200.qwen35moe.synth import SynthWeights, make_prompt  # noqa: E402

CASES = [
    # name, layers, M, prompt length, generated steps, init, fmt, router
    ("qwen35moe_l4_m2_fp8", 4, 2, 4, 4, "realistic", "fp8", "uniform"),
    ("qwen35moe_l4_m3_fp8_zipf", 4, 3, 3, 3, "realistic", "fp8", "zipf"),
    ("qwen35moe_l4_m2_bf16", 4, 2, 3, 3, "realistic", "bf16", "uniform"),      # the CPU pin test replays this one
]
VOCAB = 4096
N_PROBE = 128


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference")
    sys.path.insert(0, os.path.join(ref_root, "qwen3.6-35b-a3b-gfx942"))
    from mk import reference as R

    only = sys.argv[2] if len(sys.argv) > 2 else None
    for name, layers, M, n_prompt, n_gen, init, fmt, router in CASES:
        if only and name != only:
            continue
        t0 = time.time()
        shape = FULL.with_(vocab=VOCAB, layers=layers)
        W = SynthWeights(shape, layers=layers, seed=11, init=init, fmt=fmt, device="cpu", router=router)
        st = R.State.new(M, 64, device="cpu")
        prompts = [make_prompt(VOCAB, n_prompt, seed=j) for j in range(M)]
        gen = torch.Generator().manual_seed(99)
        probe = torch.randperm(VOCAB, generator=gen)[:N_PROBE].sort().values
        rec = {"name": name, "layers": layers, "M": M, "vocab": VOCAB, "seed": 11, "init": init, "fmt": fmt, "router": router,
               "prompts": prompts, "probe_indices": probe.tolist(), "steps": []}
        tok = None
        for t in range(n_prompt + n_gen):
            if t < n_prompt:
                tok = torch.tensor([p[t] for p in prompts])
            trace = []
            logits = R.step(W, tok, st, layers=layers, trace=trace)
            top = logits.topk(2, dim=-1).values
            tok = logits.argmax(-1)
            rec["steps"].append({"ids": tok.tolist(), "probe_logits": logits[:, probe].tolist(),
                                 "top2_gap": (top[:, 0] - top[:, 1]).tolist(),
                                 "abs_sum": logits.double().abs().sum(-1).tolist(),
                                 "experts": [tr["idx"].tolist() for tr in trace],
                                 "expert_weights": [tr["w"].tolist() for tr in trace]})
        n_att = sum(1 for i in range(layers) if shape.is_attn(i))
        rec["state"] = {"ssm_abs": [float(st.ssm[g].double().abs().sum()) for g in range(layers - n_att)],
                        "conv_abs": [float(st.conv[g].double().abs().sum()) for g in range(layers - n_att)]}
        path = os.path.join(HERE, name + ".json")
        with open(path, "w") as f:
            json.dump(rec, f)
        print(f"{name}: {os.path.getsize(path) / 1e3:.0f} kB in {time.time() - t0:.0f} s", flush=True)


if __name__ == "__main__":
    main()
