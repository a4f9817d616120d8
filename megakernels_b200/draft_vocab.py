"""Token ranking for the reduced draft head, and the acceptance it buys.

The draft head of a speculative cycle is an arg-max over the vocabulary; restricted to the K tokens the model
itself produces most often it streams K / vocab of the LM head's bytes per cycle and loses little acceptance.
This module is the tooling around that trade (the reference's `tools/draft_vocab.py` and `tools/mtp_acceptance.py`):

* `rank_from_counts(counts, vocab)`: ids by falling frequency, never-seen ids after them in id order: the
  `draft_ids` argument of `Megakernel(..., draft_vocab=K, draft_ids=...)`;
* `count_generated(generate, prompts, n)`: how often each id occurs in the model's own replies (self-distilled: no
  dataset is involved; `generate(prompt_ids, n) -> ids` is any callable, normally an engine's);
* `acceptance(engine, prompts, n)`: runs speculative cycles and reports, per draft-vocabulary size the engine was
  built with, tokens per cycle and the share of cycles whose draft was accepted.

    python -m megakernels_b200.draft_vocab --model /path/to/snapshot --conversations 600 --out draft_vocab.npy
"""

import argparse
import collections

import torch


def rank_from_counts(counts, vocab):
    """counts: {id: occurrences}.  Returns int64 ids [vocab]: most frequent first (ties by id), then the rest by id."""
    seen = sorted((i for i in counts if 0 <= i < vocab and counts[i] > 0), key=lambda i: (-counts[i], i))
    mark = torch.zeros(vocab, dtype=torch.bool)
    if seen:
        mark[torch.tensor(seen)] = True
    rest = torch.nonzero(~mark).flatten()
    return torch.cat([torch.tensor(seen, dtype=torch.int64), rest])


def count_generated(generate, prompts, n_tokens, stop_ids=()):
    counts = collections.Counter()
    for p in prompts:
        for t in generate(list(p), n_tokens):
            if t not in stop_ids:
                counts[int(t)] += 1
    return counts


def coverage(ranked, counts, k):
    """Share of the counted occurrences that fall on the first k ranked ids."""
    total = sum(counts.values())
    head = set(ranked[:k].tolist())
    return sum(c for i, c in counts.items() if i in head) / max(total, 1)


def acceptance(engine, prompts, n_tokens, temperature=0.0, seed=0):
    """Greedy speculative decoding of `n_tokens` per prompt on `engine` (built with mtp=True).  Returns a dict:
    cycles, tokens, tokens_per_cycle, accepted (share of cycles that emitted two ids)."""
    cycles = tokens = doubles = 0
    for p in prompts:
        engine.reset()
        pending = engine.prefill(list(p))
        guess, left = pending, n_tokens
        while left > 0:
            ids, guess = engine.run_spec(pending, guess, min(left, 64), temperature=temperature, seed=seed)
            for emitted, _ in engine.last_cycles:
                cycles += 1
                doubles += int(emitted == 2)
            tokens += len(ids)
            left -= len(ids)
            pending = ids[-1]
    return dict(cycles=cycles, tokens=tokens, tokens_per_cycle=tokens / max(cycles, 1), accepted=doubles / max(cycles, 1))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="local snapshot directory")
    ap.add_argument("--conversations", type=int, default=600)
    ap.add_argument("--reply-tokens", type=int, default=384)
    ap.add_argument("--keep", type=int, default=65536, help="how many ranked ids to save")
    ap.add_argument("--out", default="draft_vocab.npy")
    args = ap.parse_args()
    import random

    import numpy as np

    from .session import ChatSession
    s = ChatSession.from_snapshot(args.model, max_seq=args.reply_tokens + 512, spec=False)
    rng = random.Random(0)
    topics = ["programming", "mathematics", "history", "science", "cooking", "travel", "health", "finance", "writing", "languages"]
    kinds = ["a factual question", "a coding task", "a request for an explanation", "a request for advice", "a request to write something"]
    counts = collections.Counter()
    for _ in range(args.conversations):
        # the model writes a user request from a generic seed, then answers it in a fresh chat; only replies are counted
        ask = f"Write one message a user might send to an assistant: {rng.choice(kinds)} about {rng.choice(topics)}. Only the message."
        request = s.tok.decode(list(s.chat([{"role": "user", "content": ask}], max_new_tokens=96, temperature=0.8, seed=rng.getrandbits(31))))
        for t in s.chat([{"role": "user", "content": request}], max_new_tokens=args.reply_tokens, temperature=0.7, seed=rng.getrandbits(31)):
            counts[int(t)] += 1
    ranked = rank_from_counts(counts, s.mk.cfg.vocab)
    np.save(args.out, ranked[: args.keep].numpy().astype(np.int32))
    for k in (4096, 16384, 32768, 65536):
        print(f"first {k:6d} ids cover {100 * coverage(ranked, counts, k):.2f} % of {sum(counts.values())} generated tokens")


if __name__ == "__main__":
    main()
