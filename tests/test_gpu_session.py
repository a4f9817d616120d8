"""ChatSession on a real engine (4-layer synthetic model, byte tokenizer): streams equal direct generation, a
continued conversation reuses the state, a diverging prompt returns to a snapshot, and a state computed elsewhere
can be imported."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from megakernels_b200.config import qwen35_08b
from megakernels_b200.engine import Megakernel
from megakernels_b200.session import ChatSession, import_state
from megakernels_b200.synth import make_mtp_weights, make_weights

STOP = 3000                                   # an id the byte tokenizer never produces
HEADER = list(b"<a>")


class ByteTokenizer:
    def encode(self, text):
        return list(text.encode())

    def decode(self, ids):
        return bytes(i for i in ids if i < 256).decode(errors="replace")


@pytest.fixture(scope="module")
def parts():
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    return cfg, make_weights(cfg, 0, init="realistic"), make_mtp_weights(cfg, 0)


def engine(parts, mtp=False):
    cfg, w, wm = parts
    return Megakernel((cfg, w, wm), max_seq=256, quant="int8", mtp=mtp)


@pytest.mark.parametrize("spec", [False, True])
def test_stream_equals_direct_generation_and_continues(parts, spec):
    s = ChatSession(engine(parts, spec), ByteTokenizer(), [STOP], HEADER, spec=spec)
    prompt = list(b"<u>hello<a>")
    got = list(s.stream(prompt, max_new_tokens=12, temperature=0.0))
    ref = engine(parts)
    want = list(ref.generate(prompt, max_new_tokens=12))
    assert got == want and s.stats["prefill_tokens"] == len(prompt) - 1 and s.stats["decode_tokens"] == 12
    assert s.fed == prompt + got[:-1]
    # the next turn extends the conversation: only the new tokens are fed
    turn2 = prompt + got[:-1] + list(b"<u>more<a>")
    got2 = list(s.stream(turn2, max_new_tokens=8, temperature=0.0))
    assert s.stats["prefill_tokens"] == len(b"<u>more<a>") - 1          # all of the new turn but its last token, which opens the generation
    ref.reset()
    assert got2 == list(ref.generate(turn2, max_new_tokens=8))


def test_a_diverging_prompt_returns_to_the_snapshot(parts):
    s = ChatSession(engine(parts), ByteTokenizer(), [STOP], HEADER)
    first = list(b"<u>question one<a>an answer<u>question two<a>")
    list(s.stream(first, max_new_tokens=6, temperature=0.0))
    cut = len(b"<u>question one")
    assert len(s.snapshots) == 1 and s.snapshots[0][0] == first[:cut]      # taken just before the last complete assistant header
    # the same first turn, but the template renders the earlier reply differently: the fed tokens are not a prefix
    other = first[:cut] + list(b"<a>another answer<u>question two<a>")
    got = list(s.stream(other, max_new_tokens=6, temperature=0.0))
    assert s.stats["prefill_tokens"] == len(other) - 1 - cut               # everything behind the snapshot, nothing before it
    ref = engine(parts)
    assert got == list(ref.generate(other, max_new_tokens=6))
    # an abandoned stream leaves the ledger unknown; the next request still works (from a snapshot or from scratch)
    g = s.stream(first, max_new_tokens=6, temperature=0.0)
    next(g)
    g.close()
    assert s.fed is None
    ref.reset()
    assert list(s.stream(first, max_new_tokens=6, temperature=0.0)) == list(ref.generate(first, max_new_tokens=6))


def test_imported_state_continues_bitwise(parts):
    cfg = parts[0]
    a, b = engine(parts), engine(parts)
    tokens = list(range(40, 40 + 37))
    last = a.prefill(tokens + [7])                    # a holds the state after `tokens`
    n = len(tokens)
    n_gdn = sum(t == "linear_attention" for t in cfg.layer_types)
    n_att = cfg.n_layers - n_gdn
    conv = [a.conv_window(g) for g in range(n_gdn)]
    rec = [a.deltanet_state(g) for g in range(n_gdn)]
    kv = [a.kv_rows(i, n) for i in range(n_att)]
    import_state(b, n, conv, rec, [k for k, _ in kv], [v for _, v in kv])
    assert b.pos == n
    ia, la = a.run([last], n_generate=10, return_logits=True)
    ib, lb = b.run([last], n_generate=10, return_logits=True)
    assert ia == ib and torch.equal(la, lb)
