"""Host side of the 27B tensor-parallel path on two gloo ranks (CPU): rendezvous, the greedy choice over
vocabulary slices, the verdict reduction; and the sharding arithmetic every rank's packer relies on."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    os.environ.pop("MK_TP", None)
    from megakernels_b200.qwen27b import tp as TP
    ctx = TP.init(device="cpu")
    assert (ctx.tp, ctx.rank, ctx.main) == (world, rank, rank == 0)
    g = torch.Generator().manual_seed(5)
    full = torch.randn(3, 64, generator=g)
    full[1, 7] = full[1, 40] = 9.0                    # a tie across the two slices: the lower index wins
    full[2, 33] = full[2, 35] = 8.0                   # a tie inside rank 1's slice
    w = 64 // world
    ids = TP.next_token(ctx, full[:, rank * w:(rank + 1) * w])
    out[rank] = (ids.tolist(), TP.agree(ctx, True), TP.agree(ctx, rank == 0))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_choose_the_argmax_of_the_concatenated_logits():
    out = mp.Manager().dict()
    mp.spawn(_rank, args=(2, 29747, out), nprocs=2, join=True)
    g = torch.Generator().manual_seed(5)
    full = torch.randn(3, 64, generator=g)
    want = full.argmax(-1).tolist()
    want[1], want[2] = 7, 33
    assert out[0] == out[1] == (want, True, False)


def test_single_process_needs_no_group():
    from megakernels_b200.qwen27b import tp as TP
    old = os.environ.pop("WORLD_SIZE", None), os.environ.pop("MK_TP", None)
    try:
        ctx = TP.init(device="cpu")
    finally:
        for k, v in zip(("WORLD_SIZE", "MK_TP"), old):
            if v is not None:
                os.environ[k] = v
    assert ctx.tp == 1 and ctx.group is None
    lg = torch.tensor([[0.0, 3.0, 1.0]])
    assert TP.next_token(ctx, lg).tolist() == [1] and TP.agree(ctx, False) is False
    assert TP.merge_choices(torch.tensor([[1.0, 5.0], [1.0, 4.0]]), torch.tensor([[3.0, 2.0], [0.0, 9.0]]), 10).tolist() == [3, 2]


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_rank_widths_tile_the_model(tp):
    """Every rank's slices are disjoint and cover the model: heads, FFN columns, vocabulary; KV heads are
    replicated when there are more ranks than heads (the serving stack's layout)."""
    from megakernels_b200.qwen27b.dims import FULL, Dims
    d = Dims(FULL, tp)
    s = FULL
    assert d.nkh * tp == s.nkh and d.nvh * tp == s.nvh and d.nq * tp == s.nq
    assert d.ffn * tp == s.ffn and d.vocab * tp == s.vocab
    assert d.nkv == max(1, s.nkv // tp)
    seen = []
    for r in range(tp):
        seen += list(d.kv_heads(r))
    assert sorted(set(seen)) == list(range(s.nkv))
    assert d.inp_n == 2 * d.nkh * 128 + 2 * d.nvh * 128 + 2 * d.nvh
    assert d.qkv_n == 2 * d.nq * 256 + 2 * d.nkv * 256


def test_sharded_weights_sum_to_the_full_product():
    """Column-parallel shards concatenate, row-parallel shards add: the identity the in-kernel all-reduce relies on,
    checked on the packer's own row / column selections."""
    from megakernels_b200.qwen27b.dims import FULL
    from megakernels_b200.qwen27b.pack import Packed
    from megakernels_b200.qwen27b.synth import SynthWeights
    from megakernels_b200.stage import pack as P
    s = FULL.with_(hidden=256, ffn=512, vocab=512, layers=1, nkh=2, nvh=4, nq=4, nkv=2)
    W = SynthWeights(s, layers=1, seed=2, fmt="bf16")
    x = torch.randn(1, 512)
    full = x @ W.L(0, "mlp.down_proj.weight").float().t()
    acc = torch.zeros_like(full)
    for r in range(2):
        PK = Packed(W, "cpu", tp=2, rank=r)
        t, meta = PK.mats[(0, "down")]
        w = P.unpack_matrix(t, meta, 256)[:256]                 # this rank's K slice of the matrix
        acc += x[:, r * 256:(r + 1) * 256] @ w.t()
    assert torch.allclose(acc, full, rtol=1e-5, atol=1e-5)
