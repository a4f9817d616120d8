"""Pin of the 27B CPU oracle: against the fixture written from the reference's decoder at the model's full
widths, and against that decoder itself, bitwise, when the reference checkout is present.

The bf16-weight fixture is the one replayed here: the MXFP4 one differs only in the weights' values (the
decoder sees dequantised bf16 matrices either way, `reference.py:76-84`), costs minutes of CPU quantisation,
and is replayed on the GPU against the kernel instead."""

import json
import os
import sys

import pytest
import torch

from megakernels_b200.qwen27b.dims import FULL
from megakernels_b200.qwen27b.synth import SynthWeights, make_prompt
from oracle import qwen27b as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REFERENCE = os.environ.get("MK_REFERENCE_ROOT",
                           os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
FIXTURE = os.path.join(GOLDEN, "qwen27b_l4_m3_bf16.json")


@pytest.fixture(scope="module")
def case():
    g = json.load(open(FIXTURE))
    shape = FULL.with_(vocab=g["vocab"], layers=g["layers"])
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
        lg = O.step(shape, W, tok, st, layers=g["layers"])
        assert lg.argmax(-1).tolist() == rec["ids"], f"step {t}"
        assert torch.allclose(lg[:, probe], torch.tensor(rec["probe_logits"]), rtol=0, atol=1e-5)
        assert torch.allclose(lg.double().abs().sum(-1), torch.tensor(rec["abs_sum"], dtype=torch.float64), rtol=1e-6)
        tok = lg.argmax(-1)
    n = len(g["steps"])
    for gi, want in enumerate(g["state"]["ssm_abs"]):
        assert abs(float(st.ssm[gi].double().abs().sum()) - want) <= 1e-6 * want
        assert abs(float(st.conv[gi].double().abs().sum()) - g["state"]["conv_abs"][gi]) <= 1e-6 * g["state"]["conv_abs"][gi]
    for ai, want in enumerate(g["state"]["k_abs"]):
        assert abs(float(st.k[ai][:, :, :n].double().abs().sum()) - want) <= 1e-6 * want
        assert abs(float(st.v[ai][:, :, :n].double().abs().sum()) - g["state"]["v_abs"][ai]) <= 1e-6 * g["state"]["v_abs"][ai]


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "qwen3.8-27b-gfx942")), reason="reference checkout absent")
def test_oracle_equals_the_reference_decoder_bitwise(case):
    g, shape, W = case
    sys.path.insert(0, os.path.join(REFERENCE, "qwen3.8-27b-gfx942"))
    for k in [k for k in sys.modules if k == "mk" or k.startswith("mk.")]:
        del sys.modules[k]                      # another model's `mk` package may have been imported by an earlier test
    from mk import reference as R
    M = 2
    ref_st = R.State.new(M, 32, device="cpu")
    st = O.State(shape, M, 32, layers=g["layers"])
    for t in range(3):
        tok = torch.tensor([7 + t, 1000 + 13 * t])
        a = R.step(W, tok, ref_st, layers=g["layers"])
        b = O.step(shape, W, tok, st, layers=g["layers"])
        assert torch.equal(a, b), f"step {t}"
    n_gdn = st.ssm.shape[0]
    assert torch.equal(ref_st.ssm[:n_gdn], st.ssm) and torch.equal(ref_st.conv[:n_gdn], st.conv)
    assert torch.equal(ref_st.k[: st.k.shape[0]], st.k) and torch.equal(ref_st.v[: st.v.shape[0]], st.v)
    assert ref_st.pos.tolist() == st.pos.tolist()


def test_reduced_widths_are_self_consistent():
    """The width-parametrised restatement at a small shape: deterministic, batch rows independent."""
    s = FULL.with_(hidden=256, ffn=512, vocab=512, layers=4, nkh=2, nvh=4, nq=4, nkv=2)
    W = SynthWeights(s, layers=4, seed=1, init="realistic", fmt="bf16")
    st2, st1 = O.State(s, 2, 16, layers=4), O.State(s, 1, 16, layers=4)
    for t in range(4):
        both = O.step(s, W, torch.tensor([3 + t, 40 + t]), st2, layers=4)
        one = O.step(s, W, torch.tensor([40 + t]), st1, layers=4)
        assert torch.allclose(both[1], one[0], rtol=0, atol=1e-5)
