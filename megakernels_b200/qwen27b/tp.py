"""Tensor-parallel harness of the 27B engine: one process per GPU, ranks of one NVSwitch node.

Same surface as the reference's harness (`qwen3.8-27b-gfx942/mk/tp.py:25-130`): `init() -> Ctx`,
`packed(ctx, W)`, `engine(ctx, PK, M)`, `next_token(ctx, logits)`, `agree(ctx, ok)`, `raw(engine)`.

What crosses the links, and where:

* the residual-stream partial sums of the three row-parallel GEMVs of a layer (out / o projection, MLP down):
  inside the megakernel, tile by tile, through mailboxes in every rank's memory that the kernel writes with
  plain peer stores (`stage/runtime.py: PeerMailbox`, the all-reduce epilogue of the GEMV stage).  No library
  collective runs on the decode path;
* the greedy choice over the ranks' vocabulary slices: inside the kernel too when `generate` runs several
  steps in one launch; for single steps `next_token` merges the slices' (max, index) pairs on the host group;
* the rendezvous and the CUDA IPC handles of the mailboxes: a `gloo` group, once, at start-up.

The ranks are launched by `torchrun` (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* in the environment); `MK_TP`
overrides the world size, `MK_TP=1` or a single process gives the plain engine.
"""

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .pack import Packed


@dataclass
class Ctx:
    tp: int
    rank: int
    group: object          # a gloo group of the tp ranks (None when tp == 1)
    device: torch.device

    @property
    def main(self):
        return self.rank == 0


def init(device=None, timeout_s=600) -> Ctx:
    """Joins the process group the launcher described.  With one process (or MK_TP=1) no group is made."""
    world = int(os.environ.get("MK_TP", os.environ.get("WORLD_SIZE", "1")))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    if device is None:
        device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world == 1:
        return Ctx(1, 0, None, device)
    if world not in (2, 4, 8):
        raise ValueError(f"tensor parallelism over {world} ranks: 2, 4 or 8")
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
        group = dist.group.WORLD
    else:
        # the caller's default group may be NCCL: the handshakes below move CPU tensors and Python objects
        group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    return Ctx(world, rank, group, device)


def packed(ctx: Ctx, W, **kw) -> Packed:
    """This rank's shard of the weights, packed for the kernel."""
    return Packed(W, ctx.device, tp=ctx.tp, rank=ctx.rank, **kw)


class TPEngine:
    """One rank's `Engine` plus the host side of a checked TP step: rank 0's tokens go to every rank, every
    rank gets the full logits (the vocabulary slices in rank order), and the residual stream after the last
    layer is compared bitwise across the ranks after every step (`ranks_equal`)."""

    def __init__(self, ctx: Ctx, PK: Packed, M: int, **kw):
        from .runner import Engine
        self.ctx = ctx
        self.eng = Engine(PK, M, device=ctx.device, group=ctx.group, **kw)
        self.ranks_equal = True
        self.steps = 0

    def reset(self):
        self.eng.reset()

    def step(self, tok: torch.Tensor) -> torch.Tensor:
        g = self.ctx.group
        t = tok.to(torch.int64).cpu().contiguous()
        dist.broadcast(t, 0, group=g)
        mine = self.eng.step(t).cpu()
        self.eng.check()
        parts = [torch.empty_like(mine) for _ in range(self.ctx.tp)]
        dist.all_gather(parts, mine, group=g)
        h = self.eng.hidden().cpu().view(torch.int32).flatten()
        hs = [torch.empty_like(h) for _ in range(self.ctx.tp)]
        dist.all_gather(hs, h, group=g)
        same = all(torch.equal(hs[0], x) for x in hs[1:])
        if not same and self.ranks_equal:
            print(f"[rank {self.ctx.rank}] residual streams differ at step {self.steps}", flush=True)
        self.ranks_equal &= same
        self.steps += 1
        return torch.cat(parts, -1).to(self.ctx.device)

    def generate(self, tok: torch.Tensor, n_steps: int) -> torch.Tensor:
        """n greedy steps in one launch per rank; the choice over the vocabulary slices is made inside the kernels."""
        t = tok.to(torch.int64).cpu().contiguous()
        dist.broadcast(t, 0, group=self.ctx.group)
        return self.eng.generate(t, n_steps)

    def check(self):
        self.eng.check()

    def close(self):
        if self.eng.peer is not None:
            torch.cuda.synchronize(self.ctx.device)
            dist.barrier(group=self.ctx.group)
            self.eng.peer.close()
            self.eng.peer = None


def engine(ctx: Ctx, PK: Packed, M: int, **kw):
    if ctx.tp == 1:
        from .runner import Engine
        return Engine(PK, M, device=ctx.device, **kw)
    return TPEngine(ctx, PK, M, **kw)


def agree(ctx: Ctx, ok: bool) -> bool:
    """Every rank's verdict (all must pass)."""
    if ctx.tp == 1:
        return bool(ok)
    f = torch.tensor([int(bool(ok))], dtype=torch.int32)
    dist.all_reduce(f, op=dist.ReduceOp.MIN, group=ctx.group)
    return bool(f.item())


def raw(eng):
    """The rank's Engine (no host work per step)."""
    return eng.eng if isinstance(eng, TPEngine) else eng


def merge_choices(values: torch.Tensor, indices: torch.Tensor, slice_width: int) -> torch.Tensor:
    """values, indices [tp, M]: every rank's best logit and its index inside the rank's slice.  Returns the
    argmax of the concatenated logits: the largest value, ties going to the lowest rank (and, inside a rank,
    to the lowest index, which `max` already chose)."""
    ranks = torch.arange(values.shape[0], device=values.device)[:, None].expand_as(values)
    r = torch.where(values == values.max(0).values[None], ranks, values.shape[0]).min(0).values
    idx = indices.gather(0, r[None])[0].long()
    return idx + r * slice_width


def next_token(ctx: Ctx, logits: torch.Tensor) -> torch.Tensor:
    """Greedy tokens from the ranks' vocabulary slices: logits [M, vocab / tp] of this rank -> ids [M] (int64,
    on the logits' device), identical on every rank."""
    if ctx.tp == 1:
        return logits.argmax(-1)
    v, i = logits.max(-1)
    mine = torch.stack([v.float().cpu(), i.float().cpu()], -1).contiguous()     # indices < 2^24 are exact in fp32
    allv = [torch.empty_like(mine) for _ in range(ctx.tp)]
    dist.all_gather(allv, mine, group=ctx.group)
    allv = torch.stack(allv)
    return merge_choices(allv[:, :, 0], allv[:, :, 1], logits.shape[-1]).to(logits.device)
