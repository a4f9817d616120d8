"""Runs a fixed set of decode launches and prints a JSON object of SHA-256 digests of everything they produced
(ids, logits, recurrent state).  tests/test_gpu_chaos.py runs it once with the normal library and once with the
race-detection build (`MK_B200_LIBNAME` selects the library) and requires equal digests."""

import hashlib
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        t = t if torch.is_tensor(t) else torch.tensor(t)
        h.update(t.detach().cpu().contiguous().numpy().tobytes())
    return h.hexdigest()


def main():
    out = {}
    # ---- the 0.8B kernels: plain, speculative and batched launches of a 4-layer model
    from megakernels_b200.config import qwen35_08b
    from megakernels_b200.engine import Megakernel
    from megakernels_b200.synth import make_mtp_weights, make_prompt, make_weights
    cfg = qwen35_08b(n_layers=4, vocab=4096)
    w = make_weights(cfg, 0, init="realistic")
    prompt = make_prompt(cfg, 12)
    for quant in ("bf16", "int8"):
        mk = Megakernel((cfg, w, make_mtp_weights(cfg, 0)), max_seq=128, quant=quant, mtp=True)
        ids, logits = mk.run(prompt, n_generate=12, return_logits=True)
        out[f"run_{quant}"] = digest(ids, logits, *[mk.deltanet_state(i) for i in range(3)])
        mk.reset()
        last = mk.prefill(prompt)
        sids, _ = mk.run_spec(last, last, 12, return_logits=True)
        out[f"spec_{quant}"] = digest(sids, mk.last_logits, *[mk.deltanet_state(i) for i in range(3)])
        del mk
    mk = Megakernel((cfg, w), max_seq=128, quant="int8", batch=4)
    ids, logits = mk.run_batch([make_prompt(cfg, n, seed=20 + j) for j, n in enumerate((9, 4, 6, 2))], n_generate=8, return_logits=True)
    out["batch_int8"] = digest(*[torch.tensor(x) for x in ids], *logits)
    del mk
    # ---- the stage machine: dense hybrid with K splits, and the MoE hybrid with routed groups, eight sequences
    from megakernels_b200 import qwen27b, qwen35moe
    s27 = qwen27b.FULL.with_(hidden=1024, ffn=2048, vocab=4096, layers=4, nkh=4, nvh=12, nq=8, nkv=2)
    eng = qwen27b.Engine(qwen27b.Packed(qwen27b.SynthWeights(s27, layers=4, init="realistic", device="cuda"), "cuda"), 8, maxlen=64)
    lg = eng.prefill([qwen27b.make_prompt(s27.vocab, 5, seed=j) for j in range(8)]).clone()
    ids = eng.generate(lg.argmax(-1), 6)
    torch.cuda.synchronize()
    eng.check()
    out["stage_27b"] = digest(lg, ids, eng.logits, eng.ssm)
    del eng
    s35 = qwen35moe.FULL.with_(hidden=1024, vocab=4096, layers=4, nkh=4, nvh=8, nq=8, nkv=2, experts=128, fi=256, sfi=256)
    eng = qwen35moe.Engine(qwen35moe.Packed(qwen35moe.SynthWeights(s35, layers=4, init="realistic", device="cuda"), "cuda"), 8, maxlen=64)
    lg = eng.prefill([qwen35moe.make_prompt(s35.vocab, 5, seed=j) for j in range(8)]).clone()
    ids = eng.generate(lg.argmax(-1), 6)
    torch.cuda.synchronize()
    eng.check()
    out["stage_35b"] = digest(lg, ids, eng.logits, eng.ssm, eng.route_ids)
    from megakernels_b200 import _lib
    out["library"] = os.path.basename(_lib.LIB_PATH)
    print("CHAOS_DIGESTS " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
