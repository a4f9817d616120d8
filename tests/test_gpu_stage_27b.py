"""The 27B dense hybrid on the stage machine against the CPU oracle and the reference's fixtures.

Reduced widths keep the oracle quick; the fixtures of `tests/golden/qwen27b_*.json` are at the model's full
widths (truncated depth), written from the reference's own decoder.  Tolerances: the kernel rounds GEMV
inputs to bf16 as the reference does and accumulates in fp32 in a different order, so logits agree to
5e-2 absolute on logits of magnitude ~10, states to 1e-2 relative to their largest entry; greedy ids must
be equal wherever the reference's top-2 gap exceeds that tolerance.  KV rows are stored in bf16: a value that
rounds the other way differs by one unit in the last place (0.8 % at worst), two are allowed."""

import glob
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from megakernels_b200.qwen27b import Engine, Packed, SynthWeights, make_prompt
from megakernels_b200.qwen27b.dims import FULL
from oracle import qwen27b as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SMALL = FULL.with_(hidden=1024, ffn=2048, vocab=4096, layers=4, nkh=4, nvh=12, nq=8, nkv=2)
LOGIT_TOL = 5e-2
STATE_TOL = 1e-2
KV_TOL = 2e-2
PREFIX_TOL = 2e-2     # a stage's output given the kernel's own inputs to it, differences of earlier stages included


def rel(a, b):
    return float((a.float() - b.float()).abs().max()) / max(float(b.float().abs().max()), 1e-6)


@pytest.fixture(scope="module", params=["mxfp4", "bf16"])
def model(request):
    torch.backends.cuda.matmul.allow_tf32 = False
    W = SynthWeights(SMALL, layers=4, init="realistic", device="cuda", fmt=request.param)
    return W, Packed(W, "cuda")


def test_every_stage_prefix_matches_the_oracle(model):
    """Runs the program one stage further each time and compares what that stage wrote."""
    W, PK = model
    M = 2
    eng = Engine(PK, M, maxlen=128)
    tok = torch.tensor([make_prompt(SMALL.vocab, 1, seed=j)[0] for j in range(M)], device="cuda")
    st = O.State(SMALL, M, 128, layers=4, device="cuda")
    trace = []
    ref_logits = O.step(SMALL, W, tok, st, layers=4, trace=trace)
    names = ["embed"] + [f"{i}.{k}" for i in range(4) for k in ("in", "mix", "out", "gu", "down")] + ["lm"]
    assert eng.rt.n_stages == len(names)
    for k, name in enumerate(names, start=1):
        eng.reset()
        for t in (eng.h, eng.ssq, eng.y, eng.y2, eng.act, eng.logits):
            t.zero_()
        eng.rt.tok[:M].copy_(tok.int())
        eng.rt.launch(1, n_stages=k)
        torch.cuda.synchronize()
        eng.check()
        if name == "embed":
            got, want = eng.h, W["model.language_model.embed_tokens.weight"][tok].float()
        elif name == "lm":
            got, want = eng.logits, ref_logits
        else:
            tr, kind = trace[int(name[0])], name[2:]
            want = {"in": tr["y"], "mix": tr["y2"], "out": tr["h1"], "gu": tr["act"], "down": tr["h0"]}[kind]
            got = {"in": eng.y, "mix": eng.y2, "out": eng.h, "gu": eng.act, "down": eng.h}[kind][:, : want.shape[1]]
        assert rel(got, want) < PREFIX_TOL, f"stage {k} ({name})"


@pytest.mark.parametrize("M", [1, 3, 8])
def test_steps_track_the_oracle_and_generate_equals_stepping(model, M):
    W, PK = model
    eng = Engine(PK, M, maxlen=128)
    st = O.State(SMALL, M, 128, layers=4, device="cuda")
    prompts = [make_prompt(SMALL.vocab, 24, seed=j) for j in range(M)]
    for t in range(24):
        tok = torch.tensor([p[t] for p in prompts], device="cuda")
        got, want = eng.step(tok), O.step(SMALL, W, tok, st, layers=4)
        assert float((got - want).abs().max()) < LOGIT_TOL, f"step {t}"
        top = want.topk(2, dim=-1).values
        sure = (top[:, 0] - top[:, 1]) > 2 * LOGIT_TOL
        assert torch.equal(got.argmax(-1)[sure], want.argmax(-1)[sure])
    eng.check()
    # caches in the reference decoder's layouts
    assert eng.pos[:M].tolist() == [24] * M
    assert rel(eng.ssm, st.ssm) < STATE_TOL
    for gi in range(3):
        win = torch.stack([eng.conv_window(gi, m) for m in range(M)])
        assert rel(win, st.conv[gi]) < STATE_TOL
    for m in range(M):
        k, v = eng.kv_rows(0, m, 24)
        assert rel(k, st.k[0, m, :, :24]) < KV_TOL and rel(v, st.v[0, m, :, :24]) < KV_TOL
    # one launch for 10 greedy steps == ten single-step launches fed from the host, bitwise
    last = want.argmax(-1)
    snap = [t.clone() for t in (eng.conv, eng.ssm, eng.k_cache, eng.v_cache, eng.pos)]
    ids = eng.generate(last, 10)
    torch.cuda.synchronize()
    eng.check()
    gen_logits = eng.logits.clone()
    for dst, src in zip((eng.conv, eng.ssm, eng.k_cache, eng.v_cache, eng.pos), snap):
        dst.copy_(src)
    tok, want_ids = last, []
    for _ in range(10):
        lg = eng.step(tok)
        tok = lg.argmax(-1)
        want_ids.append(tok.clone())
    assert torch.equal(ids.long(), torch.stack(want_ids))
    assert torch.equal(gen_logits, eng.logits)


def test_prefill_in_one_launch_equals_stepping(model):
    W, PK = model
    M = 3
    prompts = [make_prompt(SMALL.vocab, 9, seed=20 + j) for j in range(M)]
    a, b = Engine(PK, M, maxlen=64), Engine(PK, M, maxlen=64)
    got = a.prefill(prompts).clone()
    for t in range(9):
        want = b.step(torch.tensor([p[t] for p in prompts], device="cuda"))
    a.check()
    assert torch.equal(got, want) and torch.equal(a.ssm, b.ssm) and a.pos[:M].tolist() == [9] * M
    with pytest.raises(ValueError):
        a.prefill(prompts[:2])


def test_serving_cache_layout_gives_the_same_bits(model):
    """[page][position][kv head][dim] pages of 16 positions (a serving stack's layout) against this kernel's own pages."""
    W, PK = model
    M = 3
    prompts = [make_prompt(SMALL.vocab, 21, seed=60 + j) for j in range(M)]
    own, srv = Engine(PK, M, maxlen=64), Engine(PK, M, maxlen=64, kv_layout="serving", kv_block=16)
    a, b = own.prefill(prompts).clone(), srv.prefill(prompts).clone()
    srv.check()
    assert torch.equal(a, b)
    for m in range(M):
        for x, y in zip(own.kv_rows(0, m, 21), srv.kv_rows(0, m, 21)):
            assert torch.equal(x, y)
    assert srv.k_cache.shape[2:] == (16, SMALL.nkv, 256)
    with pytest.raises(ValueError):
        Engine(PK, M, maxlen=64, kv_layout="serving", kv_block=24)


def test_a_padding_row_keeps_its_state_and_leaves_the_other_rows_alone(model):
    """`valid[m] = False` for one step: rows 0 and 2 compute what they would have, row 1's DeltaNet state, conv history,
    KV cache and position stay; fed the missed token in the next step, row 1 catches up bitwise."""
    W, PK = model
    M = 3
    prompts = [make_prompt(SMALL.vocab, 8, seed=80 + j) for j in range(M)]
    a, b = Engine(PK, M, maxlen=64), Engine(PK, M, maxlen=64)
    for t in range(5):
        tok = torch.tensor([p[t] for p in prompts], device="cuda")
        a.step(tok)
        b.step(tok)
    snap = {"ssm": b.ssm.clone(), "conv": b.conv.clone(), "k": b.k_cache.clone(), "v": b.v_cache.clone()}
    tok = torch.tensor([p[5] for p in prompts], device="cuda")
    la = a.step(tok).clone()
    lb = b.step(tok, valid=[True, False, True]).clone()
    b.check()
    assert torch.equal(la[[0, 2]], lb[[0, 2]])
    assert b.pos[:M].tolist() == [6, 5, 6]
    assert torch.equal(b.ssm[:, 1], snap["ssm"][:, 1]) and torch.equal(b.conv[:, 1], snap["conv"][:, 1])
    assert torch.equal(b.ssm[:, 0], a.ssm[:, 0]) and torch.equal(b.ssm[:, 2], a.ssm[:, 2])
    # row 1 wrote no KV row (its position-5 slot still holds what it held), rows 0 and 2 did
    for cache, key in ((b.k_cache, "k"), (b.v_cache, "v")):
        blk, off = int(b.bt[1][5 // b.kv_block]), 5 % b.kv_block
        assert torch.equal(cache[:, blk, :, off], snap[key][:, blk, :, off])
        blk0 = int(b.bt[0][5 // b.kv_block])
        assert not torch.equal(cache[:, blk0, :, off], snap[key][:, blk0, :, off])
    # the next step: row 1 gets the token it missed, the others move on
    nxt = torch.tensor([prompts[0][6], prompts[1][5], prompts[2][6]], device="cuda")
    lb2 = b.step(nxt).clone()
    b.check()
    assert torch.equal(lb2[1], la[1])
    assert b.pos[:M].tolist() == [7, 6, 7]


def test_three_query_heads_per_kv_head_as_a_rank_of_eight_has_them():
    """At TP 8 a rank holds 3 query heads and one (replicated) KV head: an odd number of heads per attention record."""
    shape = SMALL.with_(nq=3, nkv=1)
    W = SynthWeights(shape, layers=4, init="realistic", device="cuda", fmt="mxfp4")
    eng = Engine(Packed(W, "cuda"), 3, maxlen=256)
    st = O.State(shape, 3, 256, layers=4, device="cuda")
    prompts = [make_prompt(shape.vocab, 140, seed=70 + j) for j in range(3)]
    for t in range(140):                                   # past 128 positions: several chunks, odd and even record indices
        tok = torch.tensor([p[t] for p in prompts], device="cuda")
        got = eng.step(tok)
        if t % 20 == 19 or t >= 136:
            want = O.step(shape, W, tok, st, layers=4)
            assert float((got - want).abs().max()) < LOGIT_TOL, f"step {t}"
        else:
            O.step(shape, W, tok, st, layers=4, lm_head=False)
    eng.check()


def test_two_engines_share_one_set_of_packed_weights(model):
    W, PK = model
    a, b = Engine(PK, 2, maxlen=64), Engine(PK, 2, maxlen=64)
    tok = torch.tensor([5, 9], device="cuda")
    la = a.step(tok).clone()
    lb = b.step(tok).clone()
    assert torch.equal(la, lb)


def test_reset_returns_to_the_first_step(model):
    W, PK = model
    eng = Engine(PK, 1, maxlen=64)
    tok = torch.tensor([11], device="cuda")
    first = eng.step(tok).clone()
    for t in (3, 4, 5):
        eng.step(torch.tensor([t], device="cuda"))
    eng.reset()
    assert torch.equal(eng.step(tok), first)


FIXTURES = sorted(glob.glob(os.path.join(GOLDEN, "qwen27b_*.json")))


def test_full_width_fixtures_exist():
    assert FIXTURES, "run tests/golden/make_golden_27b.py where the reference checkout is present"


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p)[:-5] for p in FIXTURES])
def test_full_width_model_reproduces_the_reference_fixture(path):
    """The model's real widths through the kernel, against numbers the reference's decoder produced."""
    g = json.load(open(path))
    shape = FULL.with_(vocab=g["vocab"], layers=g["layers"])
    W = SynthWeights(shape, layers=g["layers"], seed=g["seed"], init=g["init"], fmt=g["fmt"], device="cuda",
                     keep_dequant=False)
    PK = Packed(W, "cuda")
    M = g["M"]
    eng = Engine(PK, M, maxlen=64)
    probe = torch.tensor(g["probe_indices"], device="cuda")
    n_prompt = len(g["prompts"][0])
    tok = None
    for t, rec in enumerate(g["steps"]):
        if t < n_prompt:
            tok = torch.tensor([p[t] for p in g["prompts"]], device="cuda")
        lg = eng.step(tok)
        want = torch.tensor(rec["probe_logits"], device="cuda")
        assert float((lg[:, probe] - want).abs().max()) < LOGIT_TOL, f"step {t}"
        got_ids, want_ids = lg.argmax(-1).tolist(), rec["ids"]
        for m in range(M):
            if rec["top2_gap"][m] > 2 * LOGIT_TOL:
                assert got_ids[m] == want_ids[m], f"step {t} sequence {m}"
        asum = lg.double().abs().sum(-1).cpu()
        assert torch.allclose(asum, torch.tensor(rec["abs_sum"], dtype=torch.float64), rtol=2e-3)
        tok = torch.tensor(want_ids, device="cuda")       # follow the reference's ids so later steps stay comparable
    eng.check()
    n = len(g["steps"])
    n_gdn = len(g["state"]["ssm_abs"])
    for gi in range(n_gdn):
        assert abs(float(eng.ssm_state(gi).double().abs().sum()) - g["state"]["ssm_abs"][gi]) <= 2e-3 * g["state"]["ssm_abs"][gi]
        win = torch.stack([eng.conv_window(gi, m) for m in range(M)])
        assert abs(float(win.double().abs().sum()) - g["state"]["conv_abs"][gi]) <= 2e-3 * g["state"]["conv_abs"][gi]
    for ai in range(len(g["state"]["k_abs"])):
        ks = sum(float(eng.kv_rows(ai, m, n)[0].double().abs().sum()) for m in range(M))
        vs = sum(float(eng.kv_rows(ai, m, n)[1].double().abs().sum()) for m in range(M))
        assert abs(ks - g["state"]["k_abs"][ai]) <= 2e-3 * g["state"]["k_abs"][ai]
        assert abs(vs - g["state"]["v_abs"][ai]) <= 2e-3 * g["state"]["v_abs"][ai]
