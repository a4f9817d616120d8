"""Speculative cycles with the MTP draft head must reproduce plain decoding bit for bit.

A cycle runs the pending token and the draft through the same per-token arithmetic as two plain
steps, so its ids (greedy, or sampled with the same seed) and its logits are identical whatever the
drafts are.  Shapes of the checks follow qwen3.5-0.8b/tests/test_spec.py:43-139 on seeded random
weights.  Random weights make the draft head's guesses almost always wrong, which exercises the
rejection path; the acceptance path is exercised by handing `run_spec` the correct draft.
"""

import pytest
import torch

from megakernels_b200.config import qwen35_08b
from megakernels_b200.quant import dequantized_weights
from megakernels_b200.synth import make_mtp_weights, make_prompt, make_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["bf16", "int8"])
def mk(request, lib_built):
    from megakernels_b200.engine import Megakernel
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    w = make_weights(cfg, 0, init="realistic")
    return Megakernel((cfg, w, make_mtp_weights(cfg)), max_seq=512, quant=request.param, mtp=True)


def prompt_of(mk, n=24, seed=0):
    return make_prompt(mk.cfg, n, seed=seed)


@pytest.mark.parametrize("temperature,chunk", [(0.0, 256), (0.0, 16), (0.8, 16)])
def test_spec_matches_plain(mk, temperature, chunk):
    for seed in range(3):
        ids = prompt_of(mk, 20 + seed, seed)
        kw = dict(max_new_tokens=64, temperature=temperature, seed=seed, chunk=chunk)
        mk.reset()
        want = list(mk.generate(ids, **kw))
        mk.reset()
        got = list(mk.generate(ids, spec=True, **kw))
        assert got == want, (seed, temperature, chunk)


def test_verify_logits_bitwise_on_rejections(mk):
    ids = prompt_of(mk)
    mk.reset()
    last = mk.prefill(ids)
    p0 = mk.pos
    want, logits = mk.run([last], n_generate=40, return_logits=True)
    mk.reset()
    mk.prefill(ids)
    got, _ = mk.run_spec(last, last, 40, return_logits=True)
    assert got == want
    p = p0
    for c, (n_new, _) in enumerate(mk.last_cycles):
        assert torch.equal(mk.last_logits[c, 0], logits[p - p0])
        if n_new == 2:
            assert torch.equal(mk.last_logits[c, 1], logits[p + 1 - p0])
        p += n_new
    assert p == mk.pos


def test_accepted_drafts_give_the_same_bits(mk):
    """Every cycle gets the correct draft, so every cycle accepts two tokens."""
    ids = prompt_of(mk, 30, 5)
    mk.reset()
    last = mk.prefill(ids)
    p0 = mk.pos
    want, logits = mk.run([last], n_generate=33, return_logits=True)
    mk.reset()
    mk.prefill(ids)
    pending, got, k = last, [], 0
    while k + 2 <= 32:
        out, _ = mk.run_spec(pending, want[k], 2, return_logits=True)      # one cycle, limit 2
        assert mk.last_cycles == [[2, want[k]]]
        assert torch.equal(mk.last_logits[0, 0], logits[k]) and torch.equal(mk.last_logits[0, 1], logits[k + 1])
        got += out
        pending = out[-1]
        k += 2
    assert got == want[:k] and mk.pos == p0 + k
    # a plain launch continues from the state the accepted cycles left behind
    assert mk.run([pending], n_generate=1) == [want[k]]


@pytest.mark.parametrize("n", [1, 2, 7])
def test_limit_and_continuation(mk, n):
    """Odd limits cut a cycle short; the state must still continue exactly."""
    ids = prompt_of(mk, 22, 1)
    mk.reset()
    last = mk.prefill(ids)
    a = mk.run([last], n_generate=n)
    full = a + mk.run([a[-1]], n_generate=12)
    mk.reset()
    mk.prefill(ids)
    b, draft = mk.run_spec(last, full[0], n)                 # the first draft is right, the limit may forbid using it
    assert b == a
    c, _ = mk.run_spec(b[-1], draft, 12)
    assert b + c[:] == full[: n + 12] or b + c == full       # c never emits more than its limit
    assert len(c) <= 12


def test_stop_on_either_slot(mk):
    ids = prompt_of(mk, 18, 2)
    mk.reset()
    last = mk.prefill(ids)
    full = mk.run([last], n_generate=20)
    for k in (0, 1, 4, 5):
        stop = full[k]
        first = full.index(stop)
        mk.reset()
        mk.prefill(ids)
        got, _ = mk.run_spec(last, full[0], 20, stop_ids=[stop])
        assert got == full[: first + 1]
        assert mk.pos == len(ids) + first          # every emitted token but the stop id has been fed


def test_drafts_follow_the_oracle_draft_head(mk):
    """The draft the kernel proposes equals the CPU oracle's MTP argmax on the same inputs, except at
    near-ties."""
    from oracle.decoder import Decoder, MtpHead, pick_token
    cfg = mk.cfg
    w = dequantized_weights(make_weights(cfg, 0, init="realistic"), mk.quant)
    wm = dequantized_weights(make_mtp_weights(cfg), mk.quant)
    dec = Decoder(cfg, w, max_seq=512)
    head = MtpHead(cfg, wm, w["embed_tokens.weight"], 512)
    ids = prompt_of(mk, 16, 3)
    mk.reset()
    last = mk.prefill(ids)
    hidden = []
    for t in ids[:-1]:
        dec.step(t)
        hidden.append(dec.last_hidden)
    head.fill_kv(torch.stack(hidden[:-1]), torch.tensor(ids[1:-1]), 0)
    pending_h = hidden[-1]                                   # entry len(ids) - 2 waits for ids[-1]
    head.fill_kv(pending_h[None], torch.tensor([last]), len(ids) - 2)
    agree = total = 0
    pending, draft = last, last
    for _ in range(24):
        pos = mk.pos
        out, next_draft = mk.run_spec(pending, draft, 1)     # one cycle, one token (limit 1)
        lg = dec.step(pending)
        assert out == [pick_token(lg)]
        mtp_logits = head.forward(dec.last_hidden[None], torch.tensor(out), pos)[0]
        top = mtp_logits.topk(2)
        if float(top.values[0] - top.values[1]) > 1e-3:
            total += 1
            agree += int(next_draft == int(top.indices[0]))
        pending, draft = out[0], next_draft
    assert total >= 12 and agree == total, (agree, total)
