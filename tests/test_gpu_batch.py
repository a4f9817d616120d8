"""Batched decoding (several sequences per pass over the weights) vs the CPU oracle, through the C ABI.

Every sequence of a batch must behave exactly like a sequence decoded alone: the oracle is run once
per sequence (the reference's batched engines are checked the same way, sequence by sequence against
`mk.reference.step`: qwen3.8-27b-gfx942/tests/test_engine.py).  Tolerances as for the single-sequence
kernel: greedy ids identical, logits 2e-2 max-abs, DeltaNet state 1e-2 relative.
"""

import pytest
import torch

from megakernels_b200.config import qwen35_08b
from megakernels_b200.quant import dequantized_weights
from megakernels_b200.synth import make_prompt, make_weights

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-2
STATE_TOL = 1e-2
LENGTHS = [70, 5, 33, 64, 65, 1, 20, 48]          # ragged; two cross a KV page (64 positions)


def engine(cfg, w, **kw):
    from megakernels_b200.engine import Megakernel
    kw.setdefault("max_seq", 256)
    kw.setdefault("quant", "int8")
    return Megakernel((cfg, w), **kw)


def oracle(cfg, w, kv_dtype="fp32", max_seq=256):
    from oracle.decoder import Decoder
    return Decoder(cfg, dequantized_weights(w, "int8"), max_seq=max_seq,
                   kv_dtype=torch.bfloat16 if kv_dtype == "bf16" else None)


@pytest.fixture(scope="module")
def tiny():
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    return cfg, make_weights(cfg, 0, init="realistic")


def prompts_for(cfg, lengths):
    return [make_prompt(cfg, n, seed=100 + j) for j, n in enumerate(lengths)]


@pytest.mark.parametrize("kv", ["fp32", "bf16"])
def test_every_sequence_matches_the_oracle(tiny, kv, lib_built):
    from oracle.decoder import pick_token
    cfg, w = tiny
    mk = engine(cfg, w, kv_dtype=kv, batch=8)
    prompts = prompts_for(cfg, LENGTHS)
    n_gen = 24
    ids, logits = mk.run_batch(prompts, n_generate=n_gen, return_logits=True)
    gdn = [i for i, t in enumerate(cfg.layer_types) if t == "linear_attention"]
    att = [i for i, t in enumerate(cfg.layer_types) if t == "full_attention"]
    for j, prompt in enumerate(prompts):
        dec = oracle(cfg, w, kv)
        for t in prompt[:-1]:
            dec.step(t)
        ref = dec.step(prompt[-1])
        assert len(ids[j]) == n_gen
        worst = 0.0
        for i, got in enumerate(ids[j]):
            worst = max(worst, float((logits[j][i].cpu() - ref).abs().max()))
            want = pick_token(ref)
            top = ref.topk(2).values
            assert got == want, f"sequence {j} step {i}: got {got}, oracle {want}, top-2 gap {float(top[0] - top[1]):.3e}"
            if i + 1 < len(ids[j]):
                ref = dec.step(got)
        assert worst < LOGIT_TOL, (j, worst)
        assert mk.bpos[j] == len(prompt) + n_gen - 1
        for g, li in enumerate(gdn):
            a, b = mk.deltanet_state(g, seq=j).cpu(), dec.state[li]
            assert float((a - b).norm() / b.norm()) < STATE_TOL, (j, g)
        n = mk.bpos[j]
        for g, li in enumerate(att):
            k, v = mk.kv_rows(g, n, seq=j)
            assert torch.allclose(k.cpu(), dec.k_cache[li][:, :n], atol=2e-2)
            assert torch.allclose(v.cpu(), dec.v_cache[li][:, :n], atol=2e-2)


@pytest.mark.parametrize("batch", [1, 3, 8])
def test_batch_equals_sequences_decoded_alone(tiny, batch, lib_built):
    """Same ids as the single-sequence kernel, whatever the batch size; logits agree to rounding."""
    cfg, w = tiny
    prompts = prompts_for(cfg, LENGTHS[:batch])
    mk = engine(cfg, w, batch=batch)
    ids, logits = mk.run_batch(prompts, n_generate=16, return_logits=True)
    for j, prompt in enumerate(prompts):
        mk.reset()
        alone, alone_logits = mk.run(prompt, n_generate=16, return_logits=True)
        assert ids[j] == alone, j
        assert float((logits[j] - alone_logits).abs().max()) < 1e-3


def test_fewer_prompts_than_the_engine_holds(tiny, lib_built):
    cfg, w = tiny
    prompts = prompts_for(cfg, LENGTHS)
    mk = engine(cfg, w, batch=8)
    full = mk.run_batch(prompts, n_generate=12)
    mk.reset()
    some = mk.run_batch(prompts[:5], n_generate=12)
    assert some == full[:5]


def test_launch_shape_invariance_and_determinism(tiny, lib_built):
    """One launch == prompt launch followed by continuation launches; repeated runs give identical bits."""
    cfg, w = tiny
    prompts = prompts_for(cfg, LENGTHS)
    mk = engine(cfg, w, batch=8)
    a, la = mk.run_batch(prompts, n_generate=20, return_logits=True)
    mk.reset()
    first = mk.run_batch(prompts, n_generate=1)
    mid = mk.run_batch([p[-1:] for p in first], n_generate=10)
    rest = mk.run_batch([p[-1:] for p in mid], n_generate=10)
    for j in range(8):
        assert (first[j] + mid[j] + rest[j])[:20] == a[j], j
    mk.reset()
    b, lb = mk.run_batch(prompts, n_generate=20, return_logits=True)
    assert a == b
    assert all(torch.equal(x, y) for x, y in zip(la, lb))


def test_stop_freezes_one_sequence_and_leaves_exact_state(tiny, lib_built):
    cfg, w = tiny
    prompts = prompts_for(cfg, LENGTHS)
    mk = engine(cfg, w, batch=8)
    full = mk.run_batch(prompts, n_generate=30)
    # a token that sequence 2 emits in the middle and, with luck, nobody else before the end
    stop = full[2][11]
    cut = [seq.index(stop) if stop in seq else None for seq in full]
    mk.reset()
    head = mk.run_batch(prompts, n_generate=30, stop_ids=[stop])
    for j in range(8):
        want = full[j] if cut[j] is None else full[j][: cut[j] + 1]
        assert head[j] == want, j
        assert mk.bpos[j] == len(prompts[j]) + len(want) - 1
    # the stopped sequences continue exactly where they stopped: feed the stop token they reported
    nxt = [[seq[-1]] for seq in head]
    tail = mk.run_batch(nxt, n_generate=5)
    mk2 = engine(cfg, w, batch=1)
    for j in range(8):
        mk2.reset()
        alone = mk2.run(prompts[j], n_generate=len(head[j]) + 5)
        assert head[j] + tail[j] == alone, j


def test_everyone_stopped_ends_the_launch_early(tiny, lib_built):
    cfg, w = tiny
    prompts = prompts_for(cfg, LENGTHS[:4])
    mk = engine(cfg, w, batch=4)
    full = mk.run_batch(prompts, n_generate=12)
    stops = [seq[3] for seq in full]
    mk.reset()
    head = mk.run_batch(prompts, n_generate=100, stop_ids=stops)
    for j in range(4):
        k = min(i for i, t in enumerate(full[j]) if t in stops)
        assert head[j] == full[j][: k + 1]


def test_sampling_is_seeded_per_sequence(tiny, lib_built):
    from oracle.decoder import sample_key
    cfg, w = tiny
    prompts = prompts_for(cfg, [16, 16, 9])
    prompts[1] = prompts[0]                          # same prompt, different sequence slot
    mk = engine(cfg, w, batch=3)
    a, la = mk.run_batch(prompts, n_generate=8, temperature=0.8, seed=7, return_logits=True)
    mk.reset()
    b = mk.run_batch(prompts, n_generate=8, temperature=0.8, seed=7)
    mk.reset()
    c = mk.run_batch(prompts, n_generate=8, temperature=0.8, seed=8)
    assert a == b and a != c
    assert a[0] != a[1]                              # the slot enters the noise
    # the choice is the oracle's rule applied to the kernel's own logits
    for j in range(3):
        pos = len(prompts[j]) - 1
        for i, tok in enumerate(a[j]):
            key = sample_key(la[j][i].cpu(), 1 / 0.8, (7 + j * 0x9E3779B9) & 0xFFFFFFFF, pos + i)
            best = key.topk(2)
            if float(best.values[0] - best.values[1]) > 1e-3:      # away from a near-tie the choice must agree
                assert tok == int(best.indices[0]), (j, i)


def test_bad_arguments_are_refused(tiny, lib_built):
    cfg, w = tiny
    with pytest.raises(ValueError):
        engine(cfg, w, quant="bf16", batch=2)
    with pytest.raises(ValueError):
        engine(cfg, w, batch=9)
    with pytest.raises(ValueError):
        engine(cfg, w, batch=8, max_seq=8192)       # 8 x 128 pages > 512
    mk = engine(cfg, w, batch=2)
    with pytest.raises(ValueError):
        mk.run_batch([[1], [2], [3]])
    with pytest.raises(ValueError):
        mk.run_batch([[1], []])
    with pytest.raises(ValueError):
        mk.run_batch([[1], [2]], n_generate=1000)


def test_full_size_batch_against_the_reference_fixture(lib_built):
    """Benchmark configuration 2 at full size (24 layers, vocab 151936, 512-token prompts), eight sequences:
    sequence 0 carries the fixture's prompt and must reproduce the reference decoder's recorded greedy ids
    and probe logits; the other sequences must equal the single-sequence kernel."""
    import json
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "cfg2_int8.json")
    g = json.load(open(path))
    cfg = qwen35_08b(n_layers=g["n_layers"], vocab=g["vocab"])
    w = make_weights(cfg, g["seed"], init=g["init"])
    n_gen = len(g["ids"])
    prompts = [g["prompt"]] + [make_prompt(cfg, len(g["prompt"]) - 7 * j, seed=500 + j) for j in range(1, 8)]
    mk = engine(cfg, w, batch=8, max_seq=len(g["prompt"]) + n_gen + 8)
    ids, logits = mk.run_batch(prompts, n_generate=n_gen, return_logits=True)
    first = next((i for i, (x, y) in enumerate(zip(ids[0], g["ids"])) if x != y), None)
    assert first is None, f"diverged at step {first}: reference top-2 gap there {g['top2_gap'][first]:.3e}"
    probe = logits[0][:, g["probe_indices"]].cpu()
    assert float((probe - torch.tensor(g["probe_logits"])).abs().max()) < LOGIT_TOL
    for j in (3, 7):
        mk.reset()
        alone, alone_logits = mk.run(prompts[j], n_generate=n_gen, return_logits=True)
        assert ids[j] == alone, j
        assert float((logits[j] - alone_logits).abs().max()) < 1e-3


def test_long_context_where_attention_chunks_grow(tiny, lib_built):
    """With eight sequences each sequence has 18 CTAs for attention, so the positions one task scans grow
    from 16 to 64 and 128 within the first thousand positions.  Ragged prompts of 500 to 900 tokens put the
    sequences in different regimes in the same pass; every sequence must equal the single-sequence kernel,
    and two of them the oracle."""
    from oracle.decoder import pick_token
    cfg, w = tiny
    lengths = [900, 577, 640, 500, 833, 576, 705, 513]
    prompts = prompts_for(cfg, lengths)
    mk = engine(cfg, w, batch=8, max_seq=1024)
    ids, logits = mk.run_batch(prompts, n_generate=12, return_logits=True)
    for j, prompt in enumerate(prompts):
        mk.reset()
        alone, alone_logits = mk.run(prompt, n_generate=12, return_logits=True)
        assert ids[j] == alone, j
        assert float((logits[j] - alone_logits).abs().max()) < 1e-3
    for j in (0, 5):
        dec = oracle(cfg, w, max_seq=1024)
        for t in prompts[j][:-1]:
            dec.step(t)
        ref = dec.step(prompts[j][-1])
        for i, got in enumerate(ids[j]):
            assert float((logits[j][i].cpu() - ref).abs().max()) < LOGIT_TOL
            assert got == pick_token(ref), (j, i)
            if i + 1 < len(ids[j]):
                ref = dec.step(got)
