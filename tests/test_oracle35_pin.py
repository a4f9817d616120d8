"""Pin of the 35B-A3B CPU oracle: against the fixture written from the reference's decoder at the model's full
widths, and against that decoder itself, bitwise, when the reference checkout is present.

The bf16-weight fixture is replayed here (the decoder sees dequantised matrices either way; quantising 3 G
expert weights to FP8 on the CPU takes minutes); the FP8 fixtures are replayed on the GPU against the kernel."""

import json
import os
import sys

import pytest
import torch

from megakernels_b200.qwen35moe.dims import FULL
from megakernels_b200.qwen35moe.synth import SynthWeights, expert_load, make_prompt
from megakernels_b200.stage import quant
from oracle import qwen35moe as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REFERENCE = os.environ.get("MK_REFERENCE_ROOT",
                           os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
FIXTURE = os.path.join(GOLDEN, "qwen35moe_l4_m2_bf16.json")
HAVE_REF = os.path.isdir(os.path.join(REFERENCE, "qwen3.6-35b-a3b-gfx942"))


@pytest.fixture(scope="module")
def case():
    g = json.load(open(FIXTURE))
    shape = FULL.with_(vocab=g["vocab"], layers=g["layers"])
    W = SynthWeights(shape, layers=g["layers"], seed=g["seed"], init=g["init"], fmt=g["fmt"], device="cpu", router=g["router"])
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
        assert [tr["idx"].tolist() for tr in trace] == rec["experts"]
        assert torch.allclose(torch.stack([tr["w"] for tr in trace]), torch.tensor(rec["expert_weights"]), rtol=0, atol=1e-6)
        tok = lg.argmax(-1)
    for gi, want in enumerate(g["state"]["ssm_abs"]):
        assert abs(float(st.ssm[gi].double().abs().sum()) - want) <= 1e-6 * want


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout absent")
def test_oracle_equals_the_reference_decoder_bitwise(case):
    g, shape, W = case
    sys.path.insert(0, os.path.join(REFERENCE, "qwen3.6-35b-a3b-gfx942"))
    for k in [k for k in sys.modules if k == "mk" or k.startswith("mk.")]:
        del sys.modules[k]                      # another model's `mk` package may have been imported by an earlier test
    from mk import reference as R
    M = 2
    ref_st = R.State.new(M, 32, device="cpu")
    st = O.State(shape, M, 32, layers=g["layers"])
    for t in range(3):
        tok = torch.tensor([9 + t, 1500 + 11 * t])
        a = R.step(W, tok, ref_st, layers=g["layers"])
        b = O.step(shape, W, tok, st, layers=g["layers"])
        assert torch.equal(a, b), f"step {t}"
    n_gdn, n_att = st.ssm.shape[0], st.k.shape[0]
    assert torch.equal(ref_st.ssm[:n_gdn], st.ssm) and torch.equal(ref_st.conv[:n_gdn], st.conv)
    assert torch.equal(ref_st.k[:n_att], st.k) and torch.equal(ref_st.v[:n_att], st.v)


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout absent")
def test_fp8_block_dequantiser_equals_the_reference():
    sys.path.insert(0, os.path.join(REFERENCE, "qwen3.6-35b-a3b-gfx942"))
    for k in [k for k in sys.modules if k == "mk" or k.startswith("mk.")]:
        del sys.modules[k]
    from mk import reference as R
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(300, 384, generator=g) * 0.05).to(torch.bfloat16)
    q, sc = quant.quantize_fp8_block(w)
    assert torch.equal(quant.dequantize_fp8_block(q, sc), R.dequant_fp8(q, sc))


def test_routing_rule_and_rounded_mode():
    logits = torch.tensor([[0.5, 2.0, 2.0, -1.0, 0.0, 1.0, 0.25, 0.75, 0.1, 0.2]])
    idx, w = O.route(logits, 8)
    assert idx[0].tolist()[:2] == [1, 2]                       # a tie goes to the lower id
    assert abs(float(w.sum()) - 1.0) < 1e-6 and float(w[0, 0]) == float(w[0, 1])
    s = FULL.with_(hidden=256, vocab=512, layers=4, nkh=2, nvh=4, nq=4, nkv=2, experts=128, fi=128, sfi=128)
    W = SynthWeights(s, layers=4, seed=1, fmt="bf16")
    a, b = O.State(s, 2, 16, layers=4), O.State(s, 2, 16, layers=4)
    tok = torch.tensor([3, 40])
    exact, rounded = O.step(s, W, tok, a, layers=4), O.step(s, W, tok, b, layers=4, round_inputs=True)
    assert 0 < float((exact - rounded).abs().max()) < 5e-2


def test_zipf_router_concentrates_the_load():
    s = FULL.with_(hidden=256, vocab=512, layers=1, nkh=2, nvh=4, nq=4, nkv=2, experts=128, fi=128, sfi=128)
    x = torch.randn(4096, 256, generator=torch.Generator().manual_seed(0))
    x = x / x.pow(2).mean(-1, keepdim=True).sqrt()
    loads = {}
    for kind in ("uniform", "zipf"):
        W = SynthWeights(s, layers=1, seed=2, fmt="bf16", router=kind)
        idx, _ = O.route(x @ W.L(0, "mlp.gate.weight").t(), 8)
        loads[kind] = expert_load(idx, 128)
    assert float(loads["uniform"].max()) < 4 / 128                       # near-uniform: nobody above 4x the mean
    assert float(loads["zipf"][:8].sum()) > 0.3 and float(loads["zipf"][:8].sum()) > 4 * float(loads["uniform"][:8].sum())
