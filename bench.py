"""Decode throughput of the megakernels on the benchmark's configurations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch B]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...        (N = 2, 4, 8)

Headline workload (configuration 3 of the benchmark definition, the one the multi-GPU axis of the metric
exists for): the 27B dense Gated-DeltaNet / gated-attention hybrid with MXFP4 weights (64 layers, hidden 5120,
vocabulary 248320, untied bf16 LM head), quantised from seeded N(0, 0.02) weights; `batch` sequences (8 by
default) whose 2048-token prompts have gone through the kernel, bf16 KV cache; one bench "step" is 256 greedy
decode steps of every sequence in ONE kernel launch per GPU.  With --gpus N the model is sharded over N
tensor-parallel ranks (strong scaling: the same job on more GPUs); the partial sums of the row-parallel
projections are all-reduced inside the kernel through peer memory, NCCL only reduces the timings.

Beside the headline, on one GPU, the line carries the same measurement at batch 1 (`cfg3_batch1`), the 0.8B
hybrid with int8 weights at batch 8 and batch 1 with a speculative-cycle leg (`cfg2_int8`), the 0.8B with bf16
weights at batch 1 (`cfg1_bf16`), and a CPU baseline.  Synthetic weights and prompts stand in for the checkpoints
and text the reference measures on.

`--impl reference` times the CPU restatement of the reference's own PyTorch decoder for the same model
(oracle/) on the host cores, on a bounded sample of the workload: a few full-width layers plus the LM head,
scaled to the model's depth.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "decode tok/s at batch 8 and batch 1, and fraction of the HBM roofline (27B MXFP4 hybrid at TP 1/2/4/8; 0.8B hybrids beside it)"
CFG3_PROMPT, CFG3_GENERATE = 2048, 256
PROMPT, GENERATE = 512, 512               # configuration 2 (0.8B int8)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, per decode step, from the ncu captures
# summarised under profiles/ (short launches at a 64-token context; the weight part does not grow with
# context, the KV part does): decode_kernel at batch 1, batch_kernel at batch 8.
NCU_DRAM_BYTES_PER_STEP = {1: (11.566718e9 + 328.967936e6) / 16, 8: (13.616476e9 + 2.931580e9) / 16}
NCU_CONTEXT = 64
# stage_kernel: dram bytes of the captured launch (8 of 64 layers, vocabulary 32768, batch 8, 8 steps) over the
# algorithmic bytes of that launch; the bench scales its own algorithmic bytes by it (the capture of the full model
# would hold 20 GB on the device under the profiler)
NCU_STAGE_TRAFFIC_RATIO = (17.065627e9 + 2.102116e9) / 18.072158208e9


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            sm.append(int(f[0]))
            mx.append(int(f[1]))
            reasons.update(n for n, v in zip(names, f[2:6]) if v == "Active")
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    return rank, world, int(os.environ.get("LOCAL_RANK", rank))


def aggregate(local_ms, local_tokens, world, device):
    """(max time over ranks in ms, tokens summed over ranks).  Works on gloo/CPU tensors too."""
    import torch.distributed as dist
    if world == 1:
        return local_ms, local_tokens
    t = torch.tensor([local_ms], dtype=torch.float64, device=device)
    n = torch.tensor([local_tokens], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(n, op=dist.ReduceOp.SUM)
    return float(t), float(n)


def roofline(bytes_per_launch, launch_s, kernel, traffic=None, **extra):
    peak, kind = measured_peak_gbs()
    achieved = bytes_per_launch / launch_s / 1e9
    r = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
         "peak_kind": f"of {kind}", "frac_of_8TBs": achieved / 8000.0, "traffic": traffic,
         "algorithmic_bytes_per_launch": bytes_per_launch, "kernel": kernel}
    r.update(extra)
    return r


# ======================================================================================================
# configuration 3: the 27B MXFP4 hybrid on the stage-machine megakernel, TP 1/2/4/8
# ======================================================================================================
def cfg3_config(batch, layers, tp, prompt=CFG3_PROMPT, generate=CFG3_GENERATE, vocab=0):
    """The `config` object both arms print: the same workload, named the same way."""
    return {"workload": f"27B dense hybrid ({layers} layers, hidden 5120, FFN 17408, vocab {vocab or 248320}), MXFP4 weights + bf16 LM head, "
                        f"batch {batch}, tensor parallel over {tp} GPU(s)",
            "batch": batch, "prompt_tokens": prompt, "decode_steps_per_bench_step": generate, "kv_dtype": "bf16",
            "parallelism": f"tp{tp}",
            "l2": "weights streamed per decode step (15.9 GB at TP 1) exceed the 126 MB L2; no flush needed"}


class Cfg3:
    """One rank's engine with the prompt context in place."""

    def __init__(self, args, ctx, batch, PK=None):
        from megakernels_b200.qwen27b import tp as TP
        from megakernels_b200.qwen27b.dims import FULL
        from megakernels_b200.qwen27b.synth import SynthWeights, make_prompt
        self.ctx, self.batch, self.layers = ctx, batch, args.layers
        self.prompt, self.generate = args.cfg3_prompt, args.cfg3_generate
        shape = FULL.with_(layers=args.layers) if args.layers != FULL.layers else FULL
        if args.vocab:
            shape = shape.with_(vocab=args.vocab)
        if PK is None:
            # drawn on the GPU: 27 G normals on the host would take minutes; every rank draws the same values
            W = SynthWeights(shape, layers=args.layers, seed=0, device=ctx.device, draw_device=ctx.device, keep_dequant=False)
            PK = TP.packed(ctx, W)
            del W
            torch.cuda.empty_cache()
        self.PK = PK
        eng = TP.engine(ctx, PK, batch, maxlen=self.prompt + self.generate + 64, spin_limit_ms=10000)
        self.eng = TP.raw(eng)
        prompts = [make_prompt(shape.vocab, self.prompt, seed=j) for j in range(batch)]
        if ctx.tp > 1:
            torch.distributed.barrier()
        self.eng.prefill(prompts)                      # the prompt goes through the kernel: one launch, `prompt` steps
        torch.cuda.synchronize()
        self.eng.check()
        self.snap = [t.clone() for t in (self.eng.conv, self.eng.ssm, self.eng.pos)]
        self.first = self.eng.rt.tok[:batch].clone()   # the greedy choice after the prompt
        self.host_tok = torch.empty(batch, dtype=torch.int32).pin_memory()
        self.host_tok.copy_(self.first.cpu())
        self.host_ids = torch.empty(self.generate, batch, dtype=torch.int32).pin_memory()
        self.launches = 0

    def restore(self):
        # positions past the prompt are simply written again, so the KV cache needs no copy
        for dst, src in zip((self.eng.conv, self.eng.ssm, self.eng.pos), self.snap):
            dst.copy_(src)

    def one_step(self):
        """One generation end to end: token ids from pinned host memory, one launch, chosen ids back to the host."""
        stream = torch.cuda.current_stream()
        self.restore()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tok = self.host_tok.to(self.ctx.device, non_blocking=True)
        e0.record(stream)
        ids = self.eng.generate(tok, self.generate)
        e1.record(stream)
        self.host_ids.copy_(ids, non_blocking=True)
        self.launches += 1
        return e0, e1

    def measure(self, steps, warmup, sampler=None):
        world = self.ctx.tp

        def barrier():
            if world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize()

        for _ in range(warmup):
            self.one_step()
        torch.cuda.synchronize()
        self.eng.check()
        if sampler:
            sampler.start()
        barrier()
        torch.cuda.profiler.start()        # a profiler given --profile-from-start off sees the timed region only
        wall0 = time.perf_counter()
        events = [self.one_step() for _ in range(steps)]
        barrier()
        wall_s = time.perf_counter() - wall0
        torch.cuda.profiler.stop()
        clocks = sampler.stop() if sampler else None
        self.eng.check()
        kernel_ms = sum(a.elapsed_time(b) for a, b in events)
        return kernel_ms, wall_s, clocks

    def report(self, kernel_ms, wall_s, steps):
        dev = self.ctx.device
        world = self.ctx.tp
        tokens = steps * self.generate * self.batch
        # every rank computes every token: the job's tokens are counted once, the time is the slowest rank's
        total_ms, _ = aggregate(kernel_ms, 0, world, dev)
        e2e_ms, _ = aggregate(wall_s * 1e3, 0, world, dev)
        bps = self.eng.bytes_per_step(self.prompt + self.generate // 2)
        launch_s = kernel_ms / steps / 1e3
        return {"value": tokens / (total_ms / 1e3), "ms_per_step": total_ms / steps,
                "median_decode_step_us": total_ms / steps / self.generate * 1e3,
                "bytes_per_decode_step_per_gpu": bps,
                "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 4 * self.batch,
                        "d2h_bytes_per_step": 4 * self.batch * self.generate},
                "roofline": roofline(bps * self.generate, launch_s, "mks::stage_kernel", traffic=NCU_STAGE_TRAFFIC_RATIO * bps * self.generate,
                                     traffic_note="ncu capture of an 8-layer, vocabulary-32768, batch-8 launch (traffic / algorithmic bytes = "
                                                  f"{NCU_STAGE_TRAFFIC_RATIO:.3f}), scaled to this launch by its algorithmic bytes",
                                     note="per GPU: this rank's weight shard, DeltaNet state and KV cache; at TP > 1 the step also "
                                          "waits for the peers' partial sums")}


def cfg3_cpu_rate(batch, n_layers=4, reps=2, vocab=None, fmt="bf16"):
    """tok/s of the CPU decoder (oracle/qwen27b.py, the restated reference) for the 27B model, estimated from a
    bounded sample: `n_layers` full-width layers (one pattern period: 3 DeltaNet + 1 attention) and the LM head are
    timed and scaled to 64 layers.  The weights are bf16 (the decoder sees dequantised matrices either way)."""
    from megakernels_b200.qwen27b.dims import FULL
    from megakernels_b200.qwen27b.synth import SynthWeights
    from oracle import qwen27b as O
    torch.set_num_threads(os.cpu_count())
    shape = FULL.with_(layers=n_layers)
    W = SynthWeights(shape, layers=n_layers, seed=0, fmt=fmt, device="cpu")
    st = O.State(shape, batch, 64, layers=n_layers)
    tok = torch.arange(batch) * 977 % shape.vocab
    body, head = [], []
    for _ in range(reps + 1):
        t0 = time.perf_counter()
        h = O.step(shape, W, tok, st, layers=n_layers, lm_head=False)
        t1 = time.perf_counter()
        x = O.rms0(h, W["model.language_model.norm.weight"], shape.eps)
        logits = x.to(torch.bfloat16).float() @ W["lm_head.weight"].float().t()
        t2 = time.perf_counter()
        tok = logits.argmax(-1)
        body.append(t1 - t0)
        head.append(t2 - t1)
    step_s = statistics.mean(body[1:]) * (FULL.layers / n_layers) + statistics.mean(head[1:])
    return batch / step_s, step_s, f"{n_layers} full-width layers (3 DeltaNet + 1 attention) and the LM head timed on a short context, " \
                                   f"scaled to {FULL.layers} layers; bf16-valued weights in fp32 arithmetic, batch {batch}"


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    rates = []
    sample = ""
    for _ in range(max(1, min(args.steps, 3))):
        rate, step_s, sample = cfg3_cpu_rate(args.batch, reps=1)
        rates.append(rate)
    value = statistics.mean(rates)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * args.batch * CFG3_GENERATE / value, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg3_config(args.batch, args.layers, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ======================================================================================================
# configurations 1 and 2: the 0.8B hybrid on the shape-specialised megakernels (one GPU)
# ======================================================================================================
def bytes_per_step(mk, batch, kv_bytes_per_pos=None):
    """Algorithmic bytes one decode step must move: every weight once, and per sequence the DeltaNet
    state read and written and the KV cache read at the average context of the generation."""
    body, head = mk.weight_bytes
    per_pos = kv_bytes_per_pos if kv_bytes_per_pos is not None else mk.kv_bytes_per_pos()
    kv = per_pos * (PROMPT + GENERATE // 2)
    return body + head + batch * (mk.state_bytes() + kv)


def build_model(quant):
    from megakernels_b200.config import qwen35_08b
    from megakernels_b200.synth import make_prompt, make_weights
    cfg = qwen35_08b()
    return cfg, make_weights(cfg, 0), make_prompt(cfg, PROMPT)


def cpu_reference_rate(cfg, w, prompt, n_prompt, n_decode, reps=1):
    """tok/s of the CPU decoder (oracle/decoder.py, the restated reference) on a bounded sample:
    `n_prompt` prompt tokens, then `n_decode` timed greedy steps."""
    from megakernels_b200.quant import dequantized_weights
    from oracle.decoder import Decoder, pick_token
    torch.set_num_threads(os.cpu_count())
    dec = Decoder(cfg, dequantized_weights(w, "int8"), max_seq=n_prompt + n_decode * reps + 1)
    logits = None
    for t in prompt[:n_prompt]:
        logits = dec.step(t)
    rates = []
    for _ in range(reps):
        t0 = time.perf_counter()
        for _ in range(n_decode):
            logits = dec.step(pick_token(logits))
        rates.append(n_decode / (time.perf_counter() - t0))
    return rates


def measure(mk, batch, prompts, args, spec=False):
    """Time `args.steps` generations of GENERATE tokens per sequence at `batch` sequences.  Returns
    (kernel ms summed over the steps, wall seconds, launches, per-decode-step ns, last run's info)."""
    stream = torch.cuda.current_stream()
    if batch == 1:
        last = [mk.prefill(prompts[0])]           # the prompt goes through the kernel, one token per step
    else:
        for i in range(0, PROMPT - 1, 512):
            mk.run_batch([p[i: min(i + 512, PROMPT - 1)] for p in prompts[:batch]])
        last = [p[-1] for p in prompts[:batch]]
    snap = mk.snapshot()
    info = {}

    def one_step(timing=False):
        mk.restore(snap)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if spec:
            got, _ = mk.run_spec(last[0], last[0], GENERATE)     # any first draft is valid; it costs at most its cycle
            info["cycles"] = len(mk.last_cycles)
            ids = [got]
        elif batch == 1:
            ids = [mk.run(last, n_generate=GENERATE, timing=timing)]
        else:
            ids = mk.run_batch([[t] for t in last], n_generate=GENERATE, timing=timing)
        e1.record(stream)
        return ids, e0, e1

    for _ in range(args.warmup):
        ids, _, _ = one_step()
    assert len(ids) == batch and all(len(x) >= GENERATE for x in ids)
    torch.cuda.synchronize()
    launches0 = mk.launches
    torch.cuda.profiler.start()            # a profiler given --profile-from-start off sees the timed region only
    wall0 = time.perf_counter()
    kernel_events, step_ns = [], []
    for _ in range(args.steps):
        ids, e0, e1 = one_step(timing=not spec)
        kernel_events.append((e0, e1))
        if not spec:
            step_ns += mk.last_step_ns
    torch.cuda.synchronize()
    wall_s = time.perf_counter() - wall0
    torch.cuda.profiler.stop()
    kernel_ms = [a.elapsed_time(b) for a, b in kernel_events]      # launch + readback of one generation
    return sum(kernel_ms), wall_s, mk.launches - launches0, step_ns, info


def report(mk, batch, kernel_ms, wall_s, step_ns, args):
    """Throughput, end-to-end throughput and roofline of one measured batch size of the 0.8B model."""
    tokens = args.steps * GENERATE * batch
    bps = bytes_per_step(mk, batch)
    launch_s = kernel_ms / args.steps / 1e3
    traffic = NCU_DRAM_BYTES_PER_STEP.get(batch)
    r = roofline(bps * GENERATE, launch_s, "mk::batch_kernel" if batch > 1 else "mk::decode_kernel",
                 traffic=traffic * GENERATE if traffic else None)
    if traffic:
        r["traffic_note"] = (f"ncu capture at a {NCU_CONTEXT}-token context scaled by decode steps: the weight and state part of a "
                             f"launch; the KV part of this {PROMPT}-token-context launch is not in it")
    # the same fraction with the KV cache counted at bf16 (2 B per element), the size the benchmark definition gives it
    bf16_kv = bytes_per_step(mk, batch, kv_bytes_per_pos=mk.kv_bytes_per_pos() * 2 // (4 if mk.kv_dtype == "fp32" else 2))
    r["frac_kv_counted_as_bf16"] = bf16_kv * GENERATE / launch_s / 1e9 / r["peak"]
    return {
        "value": tokens / (kernel_ms / 1e3), "unit": "tok/s", "ms_per_step": kernel_ms / args.steps,
        "e2e": {"value": tokens / wall_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * 8 + 4,
                "d2h_bytes_per_step": 8 * GENERATE * (8 if batch > 1 else 1) + 32 + 4},
        "median_decode_step_us": statistics.median(step_ns) / 1e3 if step_ns else None, "bytes_per_decode_step": bps,
        "roofline": r,
    }


def measure_cfg2(args, device, legs=("batch8", "batch1", "spec")):
    """int8 weights: batch 8, batch 1, and speculative cycles with the MTP draft head at batch 1."""
    from megakernels_b200.engine import Megakernel
    from megakernels_b200.synth import make_mtp_weights, make_prompt
    cfg, w, prompt = build_model("int8")
    prompts = [prompt] + [make_prompt(cfg, PROMPT, seed=1000 + j) for j in range(1, 8)]
    mk = Megakernel((cfg, w), max_seq=PROMPT + GENERATE + 64, quant="int8", kv_dtype=args.kv_dtype, device=device, batch=8)
    out = {"workload": f"qwen3.5-0.8b hybrid ({cfg.n_layers} layers, hidden 1024, vocab {cfg.vocab}), int8 per-channel weights, "
                       f"{PROMPT}-token prompt + {GENERATE} greedy steps per launch, kv {args.kv_dtype}"}
    launches, k1 = 0, None
    if "batch8" in legs:
        k8, w8, launches, s8, _ = measure(mk, 8, prompts, args)
        out["batch8"] = report(mk, 8, k8, w8, s8, args)
        mk.reset()
    if "batch1" in legs:
        k1, w1, l1, s1, _ = measure(mk, 1, prompts, args)
        out["batch1"] = report(mk, 1, k1, w1, s1, args)
        launches += l1
    del mk
    torch.cuda.empty_cache()
    if "spec" not in legs:
        return out, launches, (cfg, w, prompt)
    # speculative cycles (draft head proposes, one T = 2 pass verifies): cost of a cycle beside the plain step
    try:
        mtp = make_mtp_weights(cfg, 0)
        mk = Megakernel((cfg, w, mtp), max_seq=PROMPT + 2 * GENERATE + 64, quant="int8", kv_dtype=args.kv_dtype, device=device, mtp=True)
        ks, ws, ls, _, info = measure(mk, 1, prompts, args, spec=True)
        cycles = max(1, int(info.get("cycles", GENERATE)))
        out["spec"] = {"ms_per_cycle": ks / args.steps / cycles, "tokens_per_cycle": GENERATE / cycles,
                       "cycles_per_launch": cycles, "plain_step_ms": k1 / args.steps / GENERATE if k1 else None,
                       "value": args.steps * GENERATE / (ks / 1e3), "unit": "tok/s",
                       "note": "random weights: the draft is almost never accepted, so tokens/cycle is about 1; ms/cycle against the "
                               "plain step is what the T = 2 pass and the draft head cost"}
        launches += ls
        del mk
    except Exception as e:                                     # the leg is informative; it must not take the line down
        out["spec"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    torch.cuda.empty_cache()
    return out, launches, (cfg, w, prompt)


def measure_cfg1(args, device):
    """bf16 weights, one sequence, 32-token prompt + 128 greedy steps per bench step (one launch)."""
    global PROMPT, GENERATE
    from megakernels_b200.engine import Megakernel
    saved = PROMPT, GENERATE
    PROMPT, GENERATE = 32, 128
    try:
        cfg, w, prompt = build_model("bf16")
        mk = Megakernel((cfg, w), max_seq=PROMPT + GENERATE + 64, quant="bf16", kv_dtype=args.kv_dtype, device=device)
        kernel_ms, wall_s, launches, step_ns, _ = measure(mk, 1, [prompt], args)
        r = report(mk, 1, kernel_ms, wall_s, step_ns, args)
        r["roofline"]["traffic"] = None          # no ncu capture of the bf16 kernel is committed
        r["roofline"].pop("traffic_note", None)
        r["workload"] = "qwen3.5-0.8b hybrid, bf16 weights, batch 1, 32-token prompt + 128 greedy steps"
        return r, launches
    finally:
        PROMPT, GENERATE = saved


def measure_umma(device):
    """The block-scaled tcgen05 GEMV (`mk_umma_gemv`) on configuration 3's two largest projections, one launch per
    product, weights rotated through copies that exceed L2: what the tensor-memory path does with the matrices
    that the stage kernel streams through `mma.sync` (not part of `value`: the stage machine does not call it)."""
    from megakernels_b200.stage import umma
    peak, kind = measured_peak_gbs()
    rows = []
    for name, (r, k) in (("gate_up 34816x5120", (34816, 5120)), ("down 5120x17408", (5120, 17408))):
        for batch in (8, 1):
            m = umma.measure(r, k, batch, pieces=6, reps=20)
            rows.append({"matrix": name, "batch": batch, "us_per_launch": m["us_per_launch"], "GBs": m["gbs"],
                         "frac": m["gbs"] / peak, "peak_kind": f"of {kind}", "phases_us": m["phases_us"], "splits": m["splits"]})
    return {"kernel": "mku::gemv_kernel (tcgen05.mma kind::mxf4 block_scale, accumulators and scales in tensor memory)",
            "launches": 4 * 24, "cases": rows}


def main():
    global PROMPT, GENERATE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=8, help="sequences of the headline measurement (1..8)")
    ap.add_argument("--kv-dtype", default="fp32", choices=["fp32", "bf16"], help="KV cache of the 0.8B riders")
    ap.add_argument("--layers", type=int, default=64, help="truncate the 27B model (profiling only)")
    ap.add_argument("--vocab", type=int, default=0, help="cut the 27B model's vocabulary (profiling only)")
    ap.add_argument("--cfg3-prompt", type=int, default=CFG3_PROMPT, help="shrink the case (profiling only)")
    ap.add_argument("--cfg3-generate", type=int, default=CFG3_GENERATE, help="shrink the case (profiling only)")
    ap.add_argument("--no-riders", action="store_true", help="only the headline measurement")
    ap.add_argument("--only", default=None, choices=["cfg2", "cfg2_batch8", "cfg2_batch1", "cfg1"],
                    help="run one rider alone and print its object (profiling only; not a bench line)")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="context of the 0.8B int8 riders (profiling only)")
    ap.add_argument("--generate", type=int, default=GENERATE, help="steps per launch of the 0.8B int8 riders (profiling only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode megakernels have no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if args.only:
        PROMPT, GENERATE = args.prompt, args.generate
        if args.only == "cfg1":
            obj, _ = measure_cfg1(args, device)
        else:
            legs = ("batch8", "batch1", "spec") if args.only == "cfg2" else (args.only.split("_")[1],)
            obj, _, _ = measure_cfg2(args, device, legs)
        print(json.dumps({"only": args.only, "prompt": PROMPT, "generate": GENERATE, **obj}))
        return
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    from megakernels_b200.qwen27b import tp as TP
    ctx = TP.init(device)

    sampler = ClockSampler(local) if rank == 0 else None
    main_run = Cfg3(args, ctx, args.batch)
    kernel_ms, wall_s, clocks = main_run.measure(args.steps, args.warmup, sampler)
    head = main_run.report(kernel_ms, wall_s, args.steps)
    launches = args.steps
    riders = {}
    full_size = (args.layers, args.cfg3_prompt, args.cfg3_generate, args.vocab) == (64, CFG3_PROMPT, CFG3_GENERATE, 0)
    if world == 1 and not args.no_riders:
        if args.batch > 1:
            PK = main_run.PK
            del main_run
            torch.cuda.empty_cache()
            one = Cfg3(args, ctx, 1, PK=PK)
            k1, w1, _ = one.measure(2, 1)
            r1 = one.report(k1, w1, 2)
            riders["cfg3_batch1"] = {"value": r1["value"], "unit": "tok/s", "ms_per_step": r1["ms_per_step"],
                                     "median_decode_step_us": r1["median_decode_step_us"], "e2e": r1["e2e"],
                                     "roofline": r1["roofline"]}
            launches += 2
            del one, PK
        else:
            del main_run
        torch.cuda.empty_cache()
        if full_size:
            cfg2, l2, model = measure_cfg2(args, device)
            riders["cfg2_int8"] = cfg2
            cfg1, l1 = measure_cfg1(args, device)
            riders["cfg1_bf16"] = cfg1
            launches += l2 + l1

    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    out = {
        "metric": METRIC, "value": head["value"], "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "mxfp4 weights, bf16 activations into fp32 accumulators", "data": "synthetic",
        "config": cfg3_config(args.batch, args.layers, world, args.cfg3_prompt, args.cfg3_generate, args.vocab),
        "median_decode_step_us": head["median_decode_step_us"],
        "bytes_per_decode_step_per_gpu": head["bytes_per_decode_step_per_gpu"],
        "clocks": clocks, "e2e": head["e2e"], "gpu_launches": launches, "roofline": head["roofline"],
    }
    out.update(riders)
    if world == 1 and not args.no_riders and full_size:
        out["gpu_launches"] += 4 * 24
    if world == 1 and not args.no_riders:
        from megakernels_b200 import bw
        out["roofline"]["bw_probe_gbs"] = {m: round(bw.measure(m, gib=2.0, reps=3, device=device), 1) for m in bw.MODES}
    if world == 1 and not args.no_riders and full_size:
        out["tcgen05_mxfp4_gemv"] = measure_umma(device)
    if world == 1 and not args.no_cpu_baseline:
        rate, step_s, sample = cfg3_cpu_rate(args.batch, reps=1)
        out["cpu_baseline"] = {"value": rate, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": sample, "estimated_s_per_decode_step": step_s}
    print(json.dumps(out))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
