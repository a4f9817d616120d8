"""Pin of the 26B-A4B CPU oracle: against the fixture written from the reference's decoder at the model's full widths,
and against that decoder itself, bitwise, when the reference checkout is present (bf16-weight case here; the FP8
fixture is replayed on the GPU against the kernel, and the FP8 row-scale path is pinned live below on one layer)."""

import json
import os
import sys

import pytest
import torch

from megakernels_b200.gemma26b.dims import FULL
from megakernels_b200.gemma26b.synth import SynthWeights, make_prompt
from oracle import gemma26b as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REFERENCE = os.environ.get("MK_REFERENCE_ROOT",
                           os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
FIXTURE = os.path.join(GOLDEN, "gemma26b_l6_m2_bf16.json")
HAVE_REF = os.path.isdir(os.path.join(REFERENCE, "gemma4-26b-a4b-gfx942"))


def _reference():
    sys.path.insert(0, os.path.join(REFERENCE, "gemma4-26b-a4b-gfx942"))
    for k in [k for k in sys.modules if k == "mk" or k.startswith("mk.")]:
        del sys.modules[k]                      # another model's `mk` package may have been imported by an earlier test
    from mk import reference as R
    return R


@pytest.fixture(scope="module")
def case():
    g = json.load(open(FIXTURE))
    shape = FULL.with_(vocab=g["vocab"], layers=g["layers"], experts=g["experts"])
    W = SynthWeights(shape, layers=g["layers"], seed=g["seed"], init=g["init"], fmt=g["fmt"], device="cpu")
    return g, shape, W


def test_oracle_reproduces_the_reference_fixture(case):
    g, shape, W = case
    M, n_prompt = g["M"], len(g["prompts"][0])
    assert [make_prompt(g["vocab"], n_prompt, seed=j) for j in range(M)] == g["prompts"]
    st = O.State(shape, M, 64, layers=g["layers"])
    probe = torch.tensor(g["probe_indices"])
    tok = None
    for t, rec in enumerate(g["steps"]):
        if t < n_prompt:
            tok = torch.tensor([p[t] for p in g["prompts"]])
        trace = []
        lg = O.step(shape, W, tok, st, layers=g["layers"], trace=trace)
        assert lg.argmax(-1).tolist() == rec["ids"], f"step {t}"
        assert torch.allclose(lg[:, probe], torch.tensor(rec["probe_logits"]), rtol=0, atol=1e-5)
        assert [tr["ids"].tolist() for tr in trace] == rec["experts"]
        tok = lg.argmax(-1)


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout absent")
def test_oracle_equals_the_reference_decoder_bitwise(case):
    g, shape, W = case
    R = _reference()
    M = 2
    ref_st = R.State.new(M, 32, device="cpu")
    st = O.State(shape, M, 32, layers=g["layers"])
    for t in range(3):
        tok = torch.tensor([9 + t, 1500 + 11 * t])
        assert torch.equal(R.step(W, tok, ref_st, layers=g["layers"]), O.step(shape, W, tok, st, layers=g["layers"])), f"step {t}"
    assert torch.equal(ref_st.ks[: st.ks.shape[0]], st.ks) and torch.equal(ref_st.vf[: st.vf.shape[0]], st.vf)


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout absent")
def test_fp8_row_scaled_layer_equals_the_reference_bitwise():
    R = _reference()
    shape = FULL.with_(vocab=1024, layers=1)
    W = SynthWeights(shape, layers=1, seed=5, init="realistic", fmt="fp8", device="cpu")
    ref_st, st = R.State.new(1, 16, device="cpu"), O.State(shape, 1, 16, layers=1)
    for t in range(2):
        tok = torch.tensor([17 + t])
        assert torch.equal(R.step(W, tok, ref_st, layers=1), O.step(shape, W, tok, st, layers=1))


def test_forced_experts_keep_the_decoders_weights():
    s = FULL.with_(hidden=256, layers=1, vocab=512, nq=4, nkv_s=2, nkv_f=2, ffn=256, experts=128, eff=128, window=8)
    W = SynthWeights(s, layers=1, seed=2, fmt="bf16", init="realistic")
    tok = torch.tensor([5, 6])
    tr = []
    own = O.step(s, W, tok, O.State(s, 2, 16, layers=1), layers=1, trace=tr)
    same = O.step(s, W, tok, O.State(s, 2, 16, layers=1), layers=1, force_ids=[tr[0]["ids"]])
    other = O.step(s, W, tok, O.State(s, 2, 16, layers=1), layers=1, force_ids=[(tr[0]["ids"] + 1) % 128])
    assert torch.equal(own, same) and not torch.equal(own, other)


def test_window_limits_what_a_sliding_layer_sees():
    s = FULL.with_(hidden=256, layers=1, vocab=512, nq=4, nkv_s=2, nkv_f=2, ffn=256, experts=128, eff=128, window=4)
    W = SynthWeights(s, layers=1, seed=3, fmt="bf16", init="realistic")
    a, b = O.State(s, 1, 32, layers=1), O.State(s, 1, 32, layers=1)
    # two histories that differ only before the window
    for t in range(6):
        O.step(s, W, torch.tensor([10 + t]), a, layers=1)
        O.step(s, W, torch.tensor([(10 + t) if t >= 2 else 99]), b, layers=1)
    assert not torch.equal(a.ks[0, 0, :, :2], b.ks[0, 0, :, :2])
    la = O.step(s, W, torch.tensor([7]), a, layers=1)         # position 6 sees positions 3..6 of a single-layer model
    lb = O.step(s, W, torch.tensor([7]), b, layers=1)
    assert torch.equal(la, lb)
