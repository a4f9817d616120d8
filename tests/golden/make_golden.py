"""Write the golden fixtures in this folder from the reference's own PyTorch decoder.

Run in a checkout that has the reference project next to it:

    python tests/golden/make_golden.py /path/to/reference [case ...]

It imports `qwen_mk.reference.ReferenceModel` from `<reference>/qwen3.5-0.8b`, feeds it the seeded
synthetic weights and prompts of `megakernels_b200.synth` (for int8 cases: the dequantised
weights, as the reference's own int8 test does) and records, per case, the greedy token ids, the
top-2 logit gap of every generated step and the logits at a few fixed vocabulary indices.  The
fixtures are what pins `oracle/decoder.py` and the CUDA path on machines without the reference.
"""

import json
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from megakernels_b200.config import qwen35_08b  # noqa: E402
from megakernels_b200.quant import dequantized_weights  # noqa: E402
from megakernels_b200.synth import make_prompt, make_weights  # noqa: E402

# name: (n_layers, vocab, quant, init, prompt tokens, generated tokens)
CASES = {
    "tiny_bf16_baseline": (4, 4096, "bf16", "baseline", 12, 24),
    "tiny_bf16_realistic": (4, 4096, "bf16", "realistic", 12, 24),
    "tiny_int8_realistic": (4, 4096, "int8", "realistic", 12, 24),
    "mid_int8_baseline": (8, 8192, "int8", "baseline", 80, 48),       # crosses a KV page boundary
    "cfg1_bf16": (24, 151936, "bf16", "baseline", 32, 128),           # benchmark configuration 1
    "cfg2_int8_short": (24, 151936, "int8", "baseline", 32, 64),
    "cfg2_int8": (24, 151936, "int8", "baseline", 512, 64),           # configuration 2's prompt length
}
N_PROBE = 32


def probe_indices(vocab):
    g = torch.Generator().manual_seed(7)
    return torch.randperm(vocab, generator=g)[:N_PROBE].tolist()


def run_case(name, ref_cls):
    n_layers, vocab, quant, init, n_prompt, n_gen = CASES[name]
    cfg = qwen35_08b(n_layers=n_layers, vocab=vocab)
    w = dequantized_weights(make_weights(cfg, 0, init=init), quant)
    model = ref_cls(cfg, w, max_seq=n_prompt + n_gen + 1, device="cpu")
    prompt = make_prompt(cfg, n_prompt)
    probes = probe_indices(vocab)
    t0 = time.time()
    for t in prompt[:-1]:
        model.step(t)
    logits = model.step(prompt[-1])
    ids, gaps, probe_logits = [], [], []
    for i in range(n_gen):
        top = logits.topk(2)
        nxt = int((logits == top.values[0]).nonzero()[0, 0])   # ties -> lowest id
        ids.append(nxt)
        gaps.append(float(top.values[0] - top.values[1]))
        probe_logits.append([float(logits[j]) for j in probes])
        if i + 1 < n_gen:
            logits = model.step(nxt)
    print(f"{name}: {time.time() - t0:.1f}s, min top-2 gap {min(gaps):.3e}", flush=True)
    return dict(name=name, n_layers=n_layers, vocab=vocab, quant=quant, init=init, seed=0, prompt=prompt, ids=ids,
                top2_gap=gaps, probe_indices=probes, probe_logits=probe_logits,
                source="qwen3.5-0.8b/qwen_mk/reference.py ReferenceModel, fp32, CPU")


def main():
    ref_root = sys.argv[1]
    sys.path.insert(0, os.path.join(ref_root, "qwen3.5-0.8b"))
    from qwen_mk.reference import ReferenceModel

    torch.set_num_threads(os.cpu_count())
    for name in (sys.argv[2:] or CASES):
        with open(os.path.join(HERE, name + ".json"), "w") as f:
            json.dump(run_case(name, ReferenceModel), f)


if __name__ == "__main__":
    main()
