"""Conversations on top of the 0.8B engine: which tokens the state holds, snapshots to return to, state import.

Same surface as the reference's `ChatSession` (`qwen3.5-0.8b/qwen_mk/session.py:63-177`): `render`, `encode`,
`stream(prompt_ids, ...)` (a generator of ids that ends with a stop id if one was produced), `chat(messages, ...)`,
`stop_ids`, `stats`.  The recurrent state cannot be rolled back, so the session keeps a ledger of exactly the tokens
the state has absorbed and up to eight snapshots of it, each taken just before an assistant header; a request that
extends the ledger continues from it, any other request returns to the longest snapshot whose tokens are a prefix
of the new prompt (a chat template re-renders earlier turns slightly differently, which is the usual case).  The
KV cache needs no copy: positions before a snapshot are never overwritten.

Differences: the engine and the tokenizer are handed in (no checkpoint can be downloaded where this library is
tested; `from_snapshot` builds both from a local directory); and a long prompt's state can be imported from any
batched forward pass through `import_state` instead of being tied to one framework's cache class.
"""

import threading
import time

import torch

MAX_SNAPSHOTS = 8


def import_state(mk, n_tokens, conv_inputs, recurrent, keys, values, hidden=None, tokens=None):
    """Put the engine into the state "after `n_tokens` tokens" computed elsewhere (a batched prefill).

    conv_inputs[g]: [channels, W] the last W conv inputs of DeltaNet layer g (positions n - W .. n - 1);
    recurrent[g]:   [heads, k, v] its state in the reference decoder's layout (the engine stores [heads, v, k]);
    keys[a], values[a]: [kv heads, n, head dim] of attention layer a;
    hidden, tokens: final-normed hidden states [n, hidden] and the token list, to fill the draft head's cache.
    The reference does this for Hugging Face cache objects (`qwen_mk/session.py:37-60`)."""
    mk.reset()
    mk._enter_mode("single")
    for g, (conv, rec) in enumerate(zip(conv_inputs, recurrent)):
        mk.set_conv_window(g, conv, n_tokens)
        mk.set_deltanet_state(g, rec)
    for a, (k, v) in enumerate(zip(keys, values)):
        mk.write_kv(a, 0, k[:, :n_tokens], v[:, :n_tokens])
    mk.pos = n_tokens
    if hidden is not None and tokens is not None:
        mk.mtp_fed(0, hidden.float(), list(tokens))


class ChatSession:
    def __init__(self, engine, tokenizer, stop_ids, assistant_header, spec=False):
        """engine: a `Megakernel`; tokenizer: `.encode(text) -> ids`, `.decode(ids) -> text`, optionally
        `.apply_chat_template`; `assistant_header`: the ids that open an assistant turn."""
        self.mk, self.tok, self.spec = engine, tokenizer, spec and engine.mtp is not None
        self.stop_ids = list(stop_ids)
        self.header = list(assistant_header)
        self.fed = []              # the ledger: tokens whose effect is in the engine state (None: unknown)
        self.snapshots = []        # (token prefix, engine snapshot, pending draft-cache entry), oldest first
        self.lock = threading.Lock()
        self.stats = {}

    @classmethod
    def from_snapshot(cls, path, max_seq=32768, device="cuda", quant="int8", spec=True):
        """Engine and tokenizer from a local checkpoint directory (needs `transformers` for the tokenizer)."""
        from transformers import AutoTokenizer

        from .engine import Megakernel
        tok = AutoTokenizer.from_pretrained(path)
        mk = Megakernel(path, max_seq=max_seq, device=device, quant=quant, mtp=spec)
        stops = [tok.convert_tokens_to_ids(t) for t in ("<|im_end|>", "<|endoftext|>")]
        return cls(mk, tok, stops, tok.encode("<|im_start|>assistant\n", add_special_tokens=False), spec=spec)

    # ---- text <-> ids
    def render(self, messages, enable_thinking=False, tools=None):
        if hasattr(self.tok, "apply_chat_template"):
            return self.tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=True,
                                                enable_thinking=enable_thinking, tools=tools)
        turns = "".join(f"<|im_start|>{m['role']}\n{m.get('content') or ''}<|im_end|>\n" for m in messages)
        return turns + "<|im_start|>assistant\n"

    def encode(self, text):
        ids = self.tok.encode(text)
        return list(ids.ids if hasattr(ids, "ids") else ids)

    # ---- state
    def _remember(self):
        keep = [s for s in self.snapshots if s[0] != self.fed][-(MAX_SNAPSHOTS - 1):]
        self.snapshots = keep + [(list(self.fed), self.mk.snapshot(), self.mk.mtp_h)]

    def _return_to(self, snap):
        prefix, state, pending = snap
        self.mk.restore(state)
        self.mk.mtp_h = pending
        self.fed = list(prefix)

    def _absorb(self, tokens):
        if tokens:
            self.mk.prefill(list(tokens) + [0])            # prefill feeds all but the last: the 0 is never fed
            self.fed += list(tokens)

    def _header_before(self, ids, lo):
        """Start of the last assistant header that begins at or after `lo`, or None."""
        h, n = self.header, len(self.header)
        if not n:
            return None
        for i in range(len(ids) - n, lo - 1, -1):
            if ids[i: i + n] == h:
                return i
        return None

    def sync(self, prompt):
        """Bring the engine to the state "after prompt[:-1]".  Returns how many tokens had to be fed."""
        want = list(prompt[:-1])
        known = self.fed is not None and len(self.fed) <= len(want) and want[: len(self.fed)] == self.fed
        if not known:
            usable = [s for s in self.snapshots if len(s[0]) <= len(want) and want[: len(s[0])] == s[0]]
            if usable:
                self._return_to(max(usable, key=lambda s: len(s[0])))
            else:
                self.mk.reset()
                self.fed = []
        start = len(self.fed)
        cut = self._header_before(want, start)
        if cut is None:
            self._absorb(want[start:])
        else:
            self._absorb(want[start:cut])
            self._remember()
            self._absorb(want[cut:])
        return len(want) - start

    # ---- generation
    def stream(self, prompt_ids, max_new_tokens=512, temperature=0.7, seed=None, chunk=16):
        """Generated ids for a tokenised prompt, one by one.  Run it to the end: only then does the session know
        what the engine has absorbed (an abandoned generator leaves the ledger unknown and the next request goes
        back to a snapshot)."""
        seed = (time.time_ns() & 0x7FFFFFFF) if seed is None else seed
        with self.lock:
            t0 = time.perf_counter()
            fed_now = self.sync(prompt_ids)
            torch.cuda.synchronize(self.mk.device)
            t1 = time.perf_counter()
            produced = []
            self.fed = None
            for t in self.mk.generate([prompt_ids[-1]], max_new_tokens=max_new_tokens, temperature=temperature, seed=seed,
                                      stop_ids=self.stop_ids, chunk=chunk, spec=self.spec):
                produced.append(t)
                yield t
            # all but the last produced id have been fed (the last is a stop id, or the id chosen when the budget ran out)
            self.fed = list(prompt_ids) + produced[:-1]
            t2 = time.perf_counter()
            self.stats = dict(prefill_tokens=fed_now, prefill_s=t1 - t0, decode_tokens=len(produced), decode_s=t2 - t1,
                              decode_tok_s=len(produced) / max(t2 - t1, 1e-9))

    def chat(self, messages, enable_thinking=False, tools=None, **kw):
        """Generated ids of the reply to `messages`, stop ids left out."""
        prompt = self.encode(self.render(messages, enable_thinking=enable_thinking, tools=tools))
        for t in self.stream(prompt, **kw):
            if t not in self.stop_ids:
                yield t
