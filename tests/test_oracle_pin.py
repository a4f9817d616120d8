"""Pin the CPU oracle: against the fixtures written from the reference's own decoder, and against
that decoder itself when the reference checkout is present."""

import glob
import json
import os
import sys

import pytest
import torch

from megakernels_b200.config import qwen35_08b
from megakernels_b200.quant import dequantized_weights
from megakernels_b200.synth import make_mtp_weights, make_prompt, make_weights
from oracle.decoder import Decoder, MtpHead, mix32, pick_token, sample_key

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
# the reference checkout, when there is one: MK_REFERENCE_ROOT, or a `reference` directory beside this repository
REFERENCE = os.environ.get("MK_REFERENCE_ROOT",
                           os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
SMALL = [p for p in sorted(glob.glob(os.path.join(GOLDEN, "*.json")))          # the 0.8B model's fixtures carry "n_layers"
         if json.load(open(p)).get("n_layers", 99) <= 8]


def test_fixtures_exist():
    assert SMALL, "tests/golden holds no small fixtures; run tests/golden/make_golden.py"


@pytest.mark.parametrize("path", SMALL, ids=[os.path.basename(p)[:-5] for p in SMALL])
def test_oracle_reproduces_reference_fixture(path):
    g = json.load(open(path))
    cfg = qwen35_08b(n_layers=g["n_layers"], vocab=g["vocab"])
    w = dequantized_weights(make_weights(cfg, g["seed"], init=g["init"]), g["quant"])
    assert make_prompt(cfg, len(g["prompt"])) == g["prompt"]
    dec = Decoder(cfg, w, max_seq=len(g["prompt"]) + len(g["ids"]) + 1)
    for t in g["prompt"][:-1]:
        dec.step(t)
    logits = dec.step(g["prompt"][-1])
    for i, want in enumerate(g["ids"]):
        assert pick_token(logits) == want, f"step {i}"
        got = logits[g["probe_indices"]]
        assert torch.allclose(got, torch.tensor(g["probe_logits"][i]), rtol=0, atol=1e-5)
        top = logits.topk(2).values
        assert abs(float(top[0] - top[1]) - g["top2_gap"][i]) < 1e-5
        if i + 1 < len(g["ids"]):
            logits = dec.step(want)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "qwen3.5-0.8b")), reason="reference checkout absent")
def test_oracle_equals_reference_classes_bitwise():
    sys.path.insert(0, os.path.join(REFERENCE, "qwen3.5-0.8b"))
    from qwen_mk.mtp import MTP
    from qwen_mk.reference import ReferenceModel

    cfg = qwen35_08b(n_layers=4, vocab=2048)
    w = make_weights(cfg, 5, init="realistic")
    ref = ReferenceModel(cfg, w, max_seq=64, device="cpu")
    dec = Decoder(cfg, w, max_seq=64)
    hidden = []
    for t in make_prompt(cfg, 20):
        a, b = ref.step(t), dec.step(t)
        assert torch.equal(a, b)
        hidden.append(dec.last_hidden)
    for i in ref.state:
        assert torch.equal(ref.state[i], dec.state[i]) and torch.equal(ref.conv_hist[i], dec.conv_hist[i])
    for i in ref.k_cache:
        assert torch.equal(ref.k_cache[i], dec.k_cache[i]) and torch.equal(ref.v_cache[i], dec.v_cache[i])
    # MTP head
    wm = make_mtp_weights(cfg)
    embed = w["embed_tokens.weight"]
    r = MTP(cfg, wm, embed, 64, device="cpu")
    m = MtpHead(cfg, wm, embed, 64)
    h = torch.stack(hidden)
    nxt = torch.tensor(make_prompt(cfg, 20, seed=3))
    r.fill_kv(h[:8], nxt[:8], 0)
    m.fill_kv(h[:8], nxt[:8], 0)
    assert torch.equal(r.forward(h[8:12], nxt[8:12], 8), m.forward(h[8:12], nxt[8:12], 8))
    assert torch.equal(r.k_cache, m.k_cache)


def test_sampling_rule():
    logits = torch.tensor([0.5, 2.0, 2.0, -1.0])
    assert pick_token(logits) == 1                                   # ties -> lowest id
    g = torch.Generator().manual_seed(0)
    big = torch.randn(5000, generator=g)
    a = pick_token(big, 1 / 0.8, seed=1, pos=7)
    assert a == pick_token(big, 1 / 0.8, seed=1, pos=7)
    draws = {pick_token(big, 1 / 0.8, seed=s, pos=7) for s in range(8)}
    assert len(draws) > 1
    # known answers of the hash behind the noise (also computed by the CUDA side)
    assert mix32(0, 0, 0) == mix32(0, 0, 0) and mix32(1, 2, 3) != mix32(3, 2, 1)
    key = sample_key(big, 2.0, 3, 11)
    ids = torch.arange(5000)
    u = ((torch.tensor([mix32(3, 11, int(i)) for i in ids[:16]]) >> 8).float() + 0.5) / 16777216.0
    assert torch.allclose(key[:16], big[:16] * 2.0 - torch.log(-torch.log(u)))


def test_bf16_kv_option_is_close():
    cfg = qwen35_08b(n_layers=4, vocab=1024)
    w = make_weights(cfg, 0)
    a, b = Decoder(cfg, w, max_seq=32), Decoder(cfg, w, max_seq=32, kv_dtype=torch.bfloat16)
    for t in make_prompt(cfg, 12):
        x, y = a.step(t), b.step(t)
    assert (x - y).abs().max() < 2e-2 and not torch.equal(x, y)
