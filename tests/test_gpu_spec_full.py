"""Speculative cycles at the size the benchmark quotes (configuration 2: 24 layers, vocabulary 151936, int8
weights, MTP head drafting over the whole vocabulary), and one whole-vector logit comparison at full depth.

The small-model checks of tests/test_gpu_spec.py prove the cycle logic; this file proves that the T = 2
instantiation still reproduces plain decoding bit for bit when the LM head and the draft head each stream
155 MB per cycle, and that it emits the ids the reference's own decoder recorded in the golden fixture.
"""

import pytest
import torch

from megakernels_b200.config import qwen35_08b
from megakernels_b200.quant import dequantized_weights
from megakernels_b200.synth import make_mtp_weights, make_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def full(lib_built):
    import json
    import os
    from megakernels_b200.engine import Megakernel
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "cfg2_int8_short.json")))
    cfg = qwen35_08b(n_layers=g["n_layers"], vocab=g["vocab"])
    w = make_weights(cfg, g["seed"], init=g["init"])
    mk = Megakernel((cfg, w, make_mtp_weights(cfg)), max_seq=len(g["prompt"]) + 2 * 64 + 16, quant=g["quant"], mtp=True)
    return mk, g, w


def test_full_size_spec_equals_plain_and_the_reference_fixture(full):
    """The T=2 instantiation at the size the benchmark quotes: greedy ids equal the reference decoder's
    recorded ids, and the verify logits of every cycle are bitwise those of plain decoding; a sampled
    run (T = 0.8) gives the same ids with and without speculation
    (qwen3.5-0.8b/tests/test_spec.py:43-71)."""
    mk, g, _ = full
    n = len(g["ids"])
    mk.reset()
    last = mk.prefill(g["prompt"])
    p0 = mk.pos
    want, logits = mk.run([last], n_generate=n, return_logits=True)
    assert want == g["ids"]
    mk.reset()
    assert list(mk.generate(g["prompt"], max_new_tokens=n, spec=True, chunk=16)) == g["ids"]
    mk.reset()
    mk.prefill(g["prompt"])
    got, _ = mk.run_spec(last, last, n, return_logits=True)
    assert got == want
    p = p0
    for c, (n_new, _) in enumerate(mk.last_cycles):
        assert torch.equal(mk.last_logits[c, 0], logits[p - p0]), c
        if n_new == 2:
            assert torch.equal(mk.last_logits[c, 1], logits[p + 1 - p0]), c
        p += n_new
    for seed in (0, 1):
        kw = dict(max_new_tokens=48, temperature=0.8, seed=seed, chunk=16)
        mk.reset()
        plain = list(mk.generate(g["prompt"], **kw))
        mk.reset()
        assert list(mk.generate(g["prompt"], spec=True, **kw)) == plain, seed


def test_full_size_whole_logit_vector_against_the_oracle(full):
    """The fixtures pin 32 probe logits per step; here every one of the 151936 logits of four
    full-depth steps is compared with the CPU oracle (max-abs <= 2e-2)."""
    from oracle.decoder import Decoder
    mk, g, w = full
    dec = Decoder(mk.cfg, dequantized_weights(w, mk.quant), max_seq=64)
    prompt = g["prompt"][:12]
    mk.reset()
    ids, logits = mk.run(prompt, n_generate=4, return_logits=True)
    for t in prompt[:-1]:
        dec.step(t)
    ref = dec.step(prompt[-1])
    for i, t in enumerate(ids):
        err = float((logits[i].cpu() - ref).abs().max())
        assert err < 2e-2, (i, err)
        assert t == int(ref.argmax()), i
        if i + 1 < len(ids):
            ref = dec.step(t)
