"""CUDA megakernel vs the CPU oracle and the reference-derived fixtures, through the C ABI.

Shapes of the checks follow the reference's GPU tests, re-expressed on seeded random weights:
per-token logits and argmax (qwen3.5-0.8b/tests/test_correctness.py:24-37), launch-shape invariance
(:40-51; tests/test_int8.py:61-68), greedy continuation (:54-70), stop-token state (:73-86), seeded
sampling (:89-97), int8 against the decoder on dequantised weights (tests/test_int8.py:46-58).
Tolerances: logits 2e-2 max-abs, greedy ids identical, DeltaNet state 1e-2 relative.
"""

import glob
import json
import os

import pytest
import torch

from megakernels_b200.config import qwen35_08b
from megakernels_b200.quant import dequantized_weights
from megakernels_b200.synth import make_prompt, make_weights

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LOGIT_TOL = 2e-2
STATE_TOL = 1e-2


def engine(cfg, w, **kw):
    from megakernels_b200.engine import Megakernel
    kw.setdefault("max_seq", 256)
    return Megakernel((cfg, w), **kw)


def oracle(cfg, w, quant, kv_dtype="fp32", max_seq=256):
    from oracle.decoder import Decoder
    return Decoder(cfg, dequantized_weights(w, quant), max_seq=max_seq,
                   kv_dtype=torch.bfloat16 if kv_dtype == "bf16" else None)


@pytest.fixture(scope="module")
def tiny():
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    return cfg, make_weights(cfg, 0, init="realistic")


@pytest.mark.parametrize("quant,kv", [("bf16", "fp32"), ("int8", "fp32"), ("bf16", "bf16"), ("int8", "bf16")])
def test_logits_state_and_greedy_ids_match_oracle(tiny, quant, kv, lib_built):
    from oracle.decoder import pick_token
    cfg, w = tiny
    mk = engine(cfg, w, quant=quant, kv_dtype=kv)
    dec = oracle(cfg, w, quant, kv)
    prompt = make_prompt(cfg, 70)                       # crosses a KV page (64 positions)
    ids, logits = mk.run(prompt, n_generate=40, return_logits=True)
    for t in prompt[:-1]:
        dec.step(t)
    ref = dec.step(prompt[-1])
    worst = 0.0
    for i, got in enumerate(ids):
        worst = max(worst, float((logits[i].cpu() - ref).abs().max()))
        want = pick_token(ref)
        top = ref.topk(2).values
        assert got == want, f"step {i}: got {got}, oracle {want}, oracle top-2 gap {float(top[0] - top[1]):.3e}"
        if i + 1 < len(ids):
            ref = dec.step(got)
    assert worst < LOGIT_TOL, worst
    gdn = [i for i, t in enumerate(cfg.layer_types) if t == "linear_attention"]
    for j, li in enumerate(gdn):
        a, b = mk.deltanet_state(j).cpu(), dec.state[li]
        assert float((a - b).norm() / b.norm()) < STATE_TOL
    att = [i for i, t in enumerate(cfg.layer_types) if t == "full_attention"]
    n = mk.pos
    for j, li in enumerate(att):
        k, v = mk.kv_rows(j, n)
        assert torch.allclose(k.cpu(), dec.k_cache[li][:, :n], atol=2e-2)
        assert torch.allclose(v.cpu(), dec.v_cache[li][:, :n], atol=2e-2)


@pytest.mark.parametrize("quant", ["bf16", "int8"])
def test_launch_shape_invariance_is_bitwise(tiny, quant, lib_built):
    """The whole prompt in one launch == one launch per token, and batched all-logits == stepwise."""
    cfg, w = tiny
    mk = engine(cfg, w, quant=quant)
    prompt = make_prompt(cfg, 24)
    a = mk.run(prompt, n_generate=16)
    _, batched = (mk.reset(), mk.run(prompt, all_logits=True))[1]
    mk.reset()
    step = []
    for t in prompt[:-1]:
        step.append(mk.run([t], return_logits=True)[1])
    b, last = mk.run([prompt[-1]], n_generate=16, return_logits=True)
    step.append(last[:1])
    assert a == b
    assert torch.equal(batched, torch.cat(step))
    # three runs, identical bits (no float atomics anywhere)
    outs = []
    for _ in range(3):
        mk.reset()
        outs.append(mk.run(prompt, n_generate=8, return_logits=True)[1])
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_stop_token_leaves_exact_state(tiny, lib_built):
    cfg, w = tiny
    mk = engine(cfg, w)
    prompt = make_prompt(cfg, 16)
    full = mk.run(prompt, n_generate=40)
    stop = full[12]
    k = full.index(stop)
    mk.reset()
    head = mk.run(prompt, n_generate=40, stop_ids=[stop])
    assert head == full[: k + 1]
    assert mk.pos == len(prompt) + k
    tail = mk.run([stop], n_generate=40 - k - 1)
    assert head + tail == full


def test_sampling_is_seeded_and_follows_the_oracle_rule(tiny, lib_built):
    from oracle.decoder import sample_key
    cfg, w = tiny
    mk = engine(cfg, w)
    prompt = make_prompt(cfg, 16)
    outs = []
    for seed in (1, 1, 2):
        mk.reset()
        outs.append(mk.run(prompt, n_generate=32, temperature=0.8, seed=seed))
    assert outs[0] == outs[1] and outs[0] != outs[2]
    mk.reset()
    ids, logits = mk.run(prompt, n_generate=1, temperature=0.8, seed=5, return_logits=True)
    key = sample_key(logits[0].cpu(), 1 / 0.8, 5, len(prompt) - 1)
    best = key.topk(2)
    if float(best.values[0] - best.values[1]) > 1e-3:      # away from a near-tie the choice must agree
        assert ids[0] == int(best.indices[0])


def test_generate_prefill_and_snapshot(tiny, lib_built):
    cfg, w = tiny
    mk = engine(cfg, w)
    prompt = make_prompt(cfg, 20)
    want = mk.run(prompt, n_generate=24)
    mk.reset()
    got = list(mk.generate(prompt, max_new_tokens=24, chunk=5))
    assert got == want
    mk.reset()
    last = mk.prefill(prompt)
    snap = mk.snapshot()
    a = mk.run([last], n_generate=10)
    mk.restore(snap)
    assert mk.run([last], n_generate=10) == a


def test_shuffled_block_table_and_poisoned_pages(tiny, lib_built):
    """Paged KV: a permuted block table gives the same bits, and pages past the context are never
    read (they hold NaN) -- the pattern of gemma4-26b-a4b-gfx942/tests/test_attention.py:1-16."""
    cfg, w = tiny
    mk = engine(cfg, w, max_seq=256)
    prompt = make_prompt(cfg, 90)
    a, la = mk.run(prompt, n_generate=20, return_logits=True)
    mk.reset()
    mk.set_block_table([3, 1, 0, 2])
    for kc, vc in zip(mk.k_cache, mk.v_cache):
        kc.fill_(float("nan"))
        vc.fill_(float("nan"))
    b, lb = mk.run(prompt, n_generate=20, return_logits=True)
    assert a == b and torch.equal(la, lb)
    assert torch.isnan(mk.k_cache[0][0]).all()              # logical page 2 -> physical 0: never reached


def test_errors(tiny, lib_built):
    from megakernels_b200 import _lib
    cfg, w = tiny
    mk = engine(cfg, w, max_seq=64)
    with pytest.raises(ValueError, match="max_seq"):
        mk.run(make_prompt(cfg, 60), n_generate=10)
    with pytest.raises(ValueError):
        mk.run([])
    with pytest.raises(_lib.MkError, match="layer pointer count"):
        _lib.check(mk.lib.mk_set_params(mk._h, _lib.i64_array([0] * 5), 5, None, 0, _lib.i64_array([0]), 1))
    assert mk.run([1, 2, 3]) is not None                    # the engine is still usable afterwards
    # a launch whose fed-back steps would wait for LM-head keys that no step publishes is refused, not run into its timeout
    import ctypes
    a = _lib.LaunchArgs(forced=mk.status.data_ptr(), n_forced=2, n_steps=4, lm_from=3, start_pos=0, epoch_base=mk.epoch,
                        tokens_out=mk.status.data_ptr(), out_info=mk.status.data_ptr(), grid=mk.grid)
    assert mk.lib.mk_launch(mk._h, ctypes.byref(a), None) == _lib.MK_ERR_BADARG
    assert b"lm_from" in mk.lib.mk_last_error()
    # so is a batched launch of more sequences than the engine's per-sequence buffers were sized for
    del mk                                                  # the library has two engine slots
    one = engine(cfg, w, quant="int8", max_seq=64)
    b = _lib.BatchArgs(batch=2, n_steps=1)
    assert one.lib.mk_launch_batch(one._h, ctypes.byref(b), None) == _lib.MK_ERR_BADARG
    assert b"sized for 1" in one.lib.mk_last_error()
    with pytest.raises(ValueError):
        engine(qwen35_08b(n_layers=2).with_(hidden=2048), w)


FULL = sorted(p for p in glob.glob(os.path.join(GOLDEN, "*.json")) if "n_layers" in json.load(open(p)))     # the 0.8B model's fixtures


@pytest.mark.parametrize("path", FULL, ids=[os.path.basename(p)[:-5] for p in FULL])
def test_reference_fixture(path, lib_built):
    """Greedy ids identical for the recorded steps (64 or more at full size), probe logits within 2e-2."""
    g = json.load(open(path))
    cfg = qwen35_08b(n_layers=g["n_layers"], vocab=g["vocab"])
    w = make_weights(cfg, g["seed"], init=g["init"])
    mk = engine(cfg, w, quant=g["quant"], max_seq=len(g["prompt"]) + len(g["ids"]) + 8)
    ids, logits = mk.run(g["prompt"], n_generate=len(g["ids"]), return_logits=True)
    probe = logits[:, g["probe_indices"]].cpu()
    want = torch.tensor(g["probe_logits"])
    first = next((i for i, (x, y) in enumerate(zip(ids, g["ids"])) if x != y), None)
    assert first is None, f"diverged at step {first}: reference top-2 gap there {g['top2_gap'][first]:.3e}, " \
                          f"probe error {float((probe[first] - want[first]).abs().max()):.3e}"
    assert float((probe - want).abs().max()) < LOGIT_TOL
