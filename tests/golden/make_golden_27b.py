"""Writes tests/golden/qwen27b_*.json from the reference's own exact-mode decoder of the 27B model.

Run where the reference checkout is present (it cannot travel to a GPU machine):

    python tests/golden/make_golden_27b.py [reference root]

The reference decoder (`qwen3.8-27b-gfx942/mk/reference.py`, `step(..., emulate=False)`) fixes the model's
widths as module constants, so every fixture is at the full 27B widths (hidden 5120, FFN 17408, 48/16 DeltaNet
heads, 24/4 attention heads) with the depth truncated and the vocabulary cut to 4096 rows; the weights are the
seeded synthetic ones of `megakernels_b200.qwen27b.synth.SynthWeights` drawn on the CPU, quantised to MXFP4 and
dequantised again for the decoder, which is what the reference does with the checkpoint's tiles
(`reference.py:76-84`).

Each fixture holds, per step: the greedy ids, the logits at fixed probe columns, the gap between the two best
logits; and after the last step sums over the recurrent state and the KV rows written, so a consumer can
check the caches without the file holding them.
"""

import json
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from megakernels_b200.qwen27b.dims import FULL  # noqa: E402
from megakernels_b200.qwen27b.synth import SynthWeights, make_prompt  # noqa: E402

CASES = [
    # name, layers, M, prompt length, generated steps, init, fmt
    ("qwen27b_l4_m2_mxfp4", 4, 2, 6, 6, "realistic", "mxfp4"),
    ("qwen27b_l4_m3_bf16", 4, 3, 4, 4, "baseline", "bf16"),
]
VOCAB = 4096
N_PROBE = 128


def state_sums(st, n_gdn, n_att, npos):
    return {
        "ssm_abs": [float(st.ssm[g].double().abs().sum()) for g in range(n_gdn)],
        "conv_abs": [float(st.conv[g].double().abs().sum()) for g in range(n_gdn)],
        "k_abs": [float(st.k[a][:, :, :npos].double().abs().sum()) for a in range(n_att)],
        "v_abs": [float(st.v[a][:, :, :npos].double().abs().sum()) for a in range(n_att)],
    }


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference")
    sys.path.insert(0, os.path.join(ref_root, "qwen3.8-27b-gfx942"))
    from mk import reference as R

    torch.manual_seed(0)
    for name, layers, M, n_prompt, n_gen, init, fmt in CASES:
        t0 = time.time()
        shape = FULL.with_(vocab=VOCAB, layers=layers)
        W = SynthWeights(shape, layers=layers, seed=7, init=init, fmt=fmt, device="cpu")
        st = R.State.new(M, 64, device="cpu")
        prompts = [make_prompt(VOCAB, n_prompt, seed=j) for j in range(M)]
        gen = torch.Generator().manual_seed(99)
        probe = torch.randperm(VOCAB, generator=gen)[:N_PROBE].sort().values
        rec = {"name": name, "layers": layers, "M": M, "vocab": VOCAB, "seed": 7, "init": init, "fmt": fmt,
               "prompts": prompts, "probe_indices": probe.tolist(), "steps": []}
        tok = None
        for t in range(n_prompt + n_gen):
            if t < n_prompt:
                tok = torch.tensor([p[t] for p in prompts])
            logits = R.step(W, tok, st, layers=layers)
            top = logits.topk(2, dim=-1).values
            tok = logits.argmax(-1)
            rec["steps"].append({"ids": tok.tolist(), "probe_logits": logits[:, probe].tolist(),
                                 "top2_gap": (top[:, 0] - top[:, 1]).tolist(),
                                 "abs_sum": logits.double().abs().sum(-1).tolist()})
        n_att = sum(1 for i in range(layers) if shape.is_attn(i))
        rec["state"] = state_sums(st, layers - n_att, n_att, n_prompt + n_gen)
        path = os.path.join(HERE, name + ".json")
        with open(path, "w") as f:
            json.dump(rec, f)
        print(f"{name}: {os.path.getsize(path) / 1e3:.0f} kB in {time.time() - t0:.0f} s", flush=True)


if __name__ == "__main__":
    main()
