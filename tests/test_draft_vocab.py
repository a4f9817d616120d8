"""Draft-vocabulary tooling (CPU part): ranking, coverage, counting."""

import torch

from megakernels_b200 import draft_vocab as dv


def test_ranking_puts_frequent_ids_first_and_keeps_every_id():
    ranked = dv.rank_from_counts({5: 10, 2: 10, 9: 3, 70: 1, 200: 4}, 64)
    assert ranked[:4].tolist() == [2, 5, 9, 0]                 # ties by id; ids outside the vocabulary (70, 200) are ignored
    assert sorted(ranked.tolist()) == list(range(64)) and ranked.dtype == torch.int64
    assert dv.rank_from_counts({}, 8).tolist() == list(range(8))


def test_counts_and_coverage():
    replies = {(1, 2): [7, 7, 8, 99], (3,): [7, 9, 99]}
    counts = dv.count_generated(lambda p, n: replies[tuple(p)][:n], [[1, 2], [3]], 4, stop_ids=[99])
    assert counts == {7: 3, 8: 1, 9: 1}
    ranked = dv.rank_from_counts(counts, 16)
    assert ranked[:3].tolist() == [7, 8, 9]
    assert dv.coverage(ranked, counts, 1) == 0.6 and dv.coverage(ranked, counts, 3) == 1.0
