"""One rank of the tensor-parallel checks of the 27B engine (run by tests/test_gpu_tp.py under torchrun,
one process per GPU).  Prints `TP_OK <rank>` when every check passed on every rank."""

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from megakernels_b200.qwen27b import tp as TP  # noqa: E402
from megakernels_b200.qwen27b.dims import FULL  # noqa: E402
from megakernels_b200.qwen27b.synth import SynthWeights, make_prompt  # noqa: E402
from oracle import qwen27b as O  # noqa: E402

SMALL = FULL.with_(hidden=1024, ffn=2048, vocab=4096, layers=4, nkh=4, nvh=12, nq=8, nkv=2)


def main():
    fmt = sys.argv[1] if len(sys.argv) > 1 else "mxfp4"
    M = int(sys.argv[2]) if len(sys.argv) > 2 else 2
    torch.backends.cuda.matmul.allow_tf32 = False
    ctx = TP.init()
    dev = ctx.device
    W = SynthWeights(SMALL, layers=4, init="realistic", device=dev, fmt=fmt)
    PK = TP.packed(ctx, W)
    eng = TP.engine(ctx, PK, M, maxlen=128, spin_limit_ms=5000)
    st = O.State(SMALL, M, 128, layers=4, device=dev)
    prompts = [make_prompt(SMALL.vocab, 16, seed=j) for j in range(M)]
    ok = True
    worst = 0.0
    for t in range(16):
        tok = torch.tensor([p[t] for p in prompts], device=dev)
        full = eng.step(tok)
        want = O.step(SMALL, W, tok, st, layers=4)
        err = float((full - want).abs().max())
        worst = max(worst, err)
        ok &= err < 5e-2
        mine = TP.raw(eng).logits
        ok &= torch.equal(TP.next_token(ctx, mine), full.argmax(-1))
    ok &= eng.ranks_equal if ctx.tp > 1 else True
    # several steps in one launch: the ranks choose the same ids inside their kernels
    last = want.argmax(-1)
    r = TP.raw(eng)
    snap = [x.clone() for x in (r.conv, r.ssm, r.k_cache, r.v_cache, r.pos)]
    ids = eng.generate(last, 8)
    torch.cuda.synchronize()
    eng.check()
    for dst, src in zip((r.conv, r.ssm, r.k_cache, r.v_cache, r.pos), snap):
        dst.copy_(src)
    tok, want_ids = last, []
    for _ in range(8):
        full = eng.step(tok)
        tok = full.argmax(-1)
        want_ids.append(tok.clone())
    ok &= torch.equal(ids.long(), torch.stack(want_ids))
    ok = TP.agree(ctx, bool(ok))
    print(f"rank {ctx.rank}/{ctx.tp} fmt {fmt} M {M}: worst logit error {worst:.3e}, ranks equal {getattr(eng, 'ranks_equal', True)}", flush=True)
    if ctx.tp > 1:
        eng.close()
    if ok:
        print(f"TP_OK {ctx.rank}", flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
