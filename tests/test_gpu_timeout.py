"""The bounded waits of the stage-machine kernel: a wait that cannot be satisfied ends after the launch's spin limit,
the kernel returns, the host reads an error status naming the wait, and the same engine computes correctly again.

The wait that runs out is the all-reduce poll of a tensor-parallel rank whose peer never sends: rank 0 of a two-rank
engine runs alone, with a zeroed local buffer standing in for the peer's mailbox view (no second process, no second
GPU, nothing faults or spins without a bound)."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from megakernels_b200 import _lib
from megakernels_b200.qwen27b import Engine, Packed, SynthWeights
from megakernels_b200.qwen27b.dims import FULL
from megakernels_b200.stage import desc as D

SMALL = FULL.with_(hidden=1024, ffn=2048, vocab=4096, layers=4, nkh=4, nvh=12, nq=8, nkv=2)


class SilentPeer:
    """Mailbox views of a rank whose peer never writes: own mailbox and a second zeroed buffer."""

    def __init__(self, device):
        n = D.query("MAILBOX_BYTES")
        self.buffers = [torch.zeros(n // 8, dtype=torch.int64, device=device) for _ in range(2)]
        self.addresses = [b.data_ptr() for b in self.buffers]

    def close(self):
        pass


def test_a_wait_that_cannot_be_satisfied_ends_with_an_error_status():
    W = SynthWeights(SMALL, layers=4, init="realistic", device="cuda")
    eng = Engine(Packed(W, "cuda", tp=2, rank=0), 1, maxlen=64, spin_limit_ms=20, mailbox=SilentPeer("cuda"))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eng.step(torch.tensor([5], device="cuda"))
    e1.record()
    torch.cuda.synchronize()
    assert e0.elapsed_time(e1) < 2000.0                       # the grid unwinds once the first wait has run out
    status = eng.rt.status.tolist()
    assert status[0] != 0 and status[1] > 0                   # an error code and the wait site
    with pytest.raises(_lib.MkError) as err:
        eng.check()
    assert err.value.code == _lib.MK_ERR_TIMEOUT and "site" in str(err.value)
    # the context is intact: a one-rank engine on the same weights' full model still computes, and so does this
    # device after the failed launch
    W1 = Packed(W, "cuda")
    good = Engine(W1, 1, maxlen=64)
    a = good.step(torch.tensor([5], device="cuda")).clone()
    good.check()
    again = Engine(W1, 1, maxlen=64)
    assert torch.equal(a, again.step(torch.tensor([5], device="cuda")))
    assert torch.isfinite(a).all()
