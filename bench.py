"""Decode throughput of the megakernel on the benchmark's int8 0.8B configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch B]

Workload (configuration 2 of the benchmark definition): the 0.8B Gated-DeltaNet / attention hybrid,
vocab 151936, int8 per-channel weights quantised from seeded N(0, 0.02) bf16 weights; every sequence
has a 512-token uniform-random prompt already in its recurrent state and KV cache, then takes 512
greedy decode steps.  The configuration is measured at batch 8 (the headline value: eight sequences
per pass over the weights, `Megakernel.run_batch`) and at batch 1 (reported beside it under
"batch1": the single-sequence kernel, `Megakernel.run`).  One bench "step" is one such generation of
512 tokens per sequence: one kernel launch.  Synthetic weights and prompts stand in for the
checkpoint and text the reference measures on.

The 0.8B model is not sharded: with --gpus N every rank runs an independent replica (weak scaling)
and the value is the sum over ranks divided by the slowest rank's time.

`--impl reference` times the CPU restatement of the reference's own PyTorch decoder (oracle/) on the
host cores, on a bounded sample of the same workload.
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

METRIC = "decode tok/s at batch 8 and batch 1 (0.8B hybrid, int8 per-channel, 512-token prompt + 512 greedy steps)"
PROMPT, GENERATE = 512, 512
L2_BYTES = 126e6
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, per decode step, from the ncu captures
# summarised under profiles/ (short launches at a short context, scaled by steps; the KV part grows with
# context, the weight part does not): decode_kernel at batch 1, batch_kernel at batch 8.
NCU_DRAM_BYTES_PER_STEP = {1: (11.604932e9 + 394.075904e6) / 16, 8: (13.618422e9 + 3.158837e9) / 16}


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


def bytes_per_step(mk, batch):
    """Algorithmic bytes one decode step must move: every weight once, and per sequence the DeltaNet
    state read and written and the KV cache read at the average context of the generation."""
    body, head = mk.weight_bytes
    kv = mk.kv_bytes_per_pos() * (PROMPT + GENERATE // 2)
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


def workload_config(quant, batch, kv_dtype, vocab, layers):
    """The `config` object both arms print: the same workload, named the same way."""
    return {"workload": f"qwen3.5-0.8b hybrid ({layers} layers, hidden 1024, vocab {vocab}), "
                        f"{quant} weights, batch {batch}, replicas only",
            "batch": batch, "prompt_tokens": PROMPT, "decode_steps_per_bench_step": GENERATE, "kv_dtype": kv_dtype,
            "l2": "weights streamed per decode step (0.65 GB int8) exceed the 126 MB L2; no flush needed"}


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    cfg, w, prompt = build_model("int8")
    n_prompt, n_decode = 32, 16
    rates = cpu_reference_rate(cfg, w, prompt, n_prompt, n_decode, reps=args.warmup + args.steps)[args.warmup:]
    value = statistics.mean(rates)
    sample = f"{n_prompt}-token prompt then {n_decode} greedy decode steps per bench step, full depth and vocabulary"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * n_decode / value, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config("int8", args.batch, "fp32", cfg.vocab, cfg.n_layers),
                       note="the CPU decoder takes the sequences of a batch one after another: its tok/s does not depend on the batch"),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def measure(mk, batch, prompts, args, world, device, sampler=None):
    """Time `args.steps` generations of GENERATE tokens per sequence at `batch` sequences.  Returns
    (kernel ms summed over the steps, wall seconds, launches, per-decode-step ns, clock record)."""
    stream = torch.cuda.current_stream()
    if batch == 1:
        last = [mk.prefill(prompts[0])]           # the prompt goes through the kernel, one token per step
    else:
        for i in range(0, PROMPT - 1, 512):
            mk.run_batch([p[i: min(i + 512, PROMPT - 1)] for p in prompts[:batch]])
        last = [p[-1] for p in prompts[:batch]]
    snap = mk.snapshot()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def one_step(timing=False):
        mk.restore(snap)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if batch == 1:
            ids = [mk.run(last, n_generate=GENERATE, timing=timing)]
        else:
            ids = mk.run_batch([[t] for t in last], n_generate=GENERATE, timing=timing)
        e1.record(stream)
        return ids, e0, e1

    for _ in range(args.warmup):
        ids, _, _ = one_step()
    assert len(ids) == batch and all(len(x) == GENERATE for x in ids)
    # ---- timed region: kernel time with inputs resident (CUDA events on the launching stream)
    if sampler:
        sampler.start()
    barrier()
    launches0 = mk.launches
    wall0 = time.perf_counter()
    kernel_events, step_ns = [], []
    for _ in range(args.steps):
        ids, e0, e1 = one_step(timing=True)
        kernel_events.append((e0, e1))
        step_ns += mk.last_step_ns
    barrier()
    wall_s = time.perf_counter() - wall0
    clocks = sampler.stop() if sampler else None
    kernel_ms = [a.elapsed_time(b) for a, b in kernel_events]      # launch + readback of one generation
    return sum(kernel_ms), wall_s, mk.launches - launches0, step_ns, clocks


def report(mk, batch, kernel_ms, wall_s, step_ns, args, world, device):
    """Throughput, end-to-end throughput and roofline of one measured batch size."""
    tokens = args.steps * GENERATE * batch
    total_ms, total_tokens = aggregate(kernel_ms, tokens, world, device)
    e2e_ms, _ = aggregate(wall_s * 1e3, tokens, world, device)
    peak, peak_kind = measured_peak_gbs()
    bps = bytes_per_step(mk, batch)
    launch_s = kernel_ms / args.steps / 1e3
    achieved = bps * GENERATE / launch_s / 1e9
    traffic = NCU_DRAM_BYTES_PER_STEP.get(batch)
    return {
        "value": total_tokens / (total_ms / 1e3), "ms_per_step": total_ms / args.steps,
        "e2e": {"value": total_tokens / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 4 * 8 + 4,
                "d2h_bytes_per_step": 8 * GENERATE * (8 if batch > 1 else 1) + 32 + 4},
        "median_decode_step_us": statistics.median(step_ns) / 1e3, "bytes_per_decode_step": bps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8TBs": achieved / 8000.0,
                     "traffic": traffic * GENERATE if traffic else None,
                     "algorithmic_bytes_per_launch": bps * GENERATE,
                     "kernel": "batch_kernel" if batch > 1 else "decode_kernel"},
    }


def measure_cfg1(args, device):
    """bf16 weights, one sequence, 32-token prompt + 128 greedy steps per bench step (one launch)."""
    global PROMPT, GENERATE
    from megakernels_b200.engine import Megakernel
    saved = PROMPT, GENERATE
    PROMPT, GENERATE = 32, 128
    try:
        cfg, w, prompt = build_model("bf16")
        mk = Megakernel((cfg, w), max_seq=PROMPT + GENERATE + 64, quant="bf16", kv_dtype=args.kv_dtype, device=device)
        kernel_ms, wall_s, _, step_ns, _ = measure(mk, 1, [prompt], args, 1, device)
        r = report(mk, 1, kernel_ms, wall_s, step_ns, args, 1, device)
        r["roofline"]["traffic"] = None          # no ncu capture of the bf16 kernel is committed
        return {"workload": "bf16 weights, batch 1, 32-token prompt + 128 greedy steps", "value": r["value"], "unit": "tok/s",
                "ms_per_step": r["ms_per_step"], "median_decode_step_us": r["median_decode_step_us"],
                "bytes_per_decode_step": r["bytes_per_decode_step"], "e2e": r["e2e"], "roofline": r["roofline"]}
    finally:
        PROMPT, GENERATE = saved


def main():
    global PROMPT, GENERATE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--quant", default="int8", choices=["int8", "bf16"])
    ap.add_argument("--kv-dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--batch", type=int, default=8, help="sequences of the headline measurement (1..8; bf16 weights: 1)")
    ap.add_argument("--no-batch1", action="store_true", help="skip the batch-1 measurement beside a batched headline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cfg1", action="store_true", help="skip the bf16 configuration-1 measurement reported beside the headline")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="shrink the case (profiling only)")
    ap.add_argument("--generate", type=int, default=GENERATE, help="shrink the case (profiling only)")
    args = ap.parse_args()
    PROMPT, GENERATE = args.prompt, args.generate
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)
    if args.quant != "int8":
        args.batch = 1

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode megakernel has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    from megakernels_b200.engine import Megakernel
    from megakernels_b200.synth import make_prompt
    cfg, w, prompt = build_model(args.quant)
    prompts = [prompt] + [make_prompt(cfg, PROMPT, seed=1000 + j) for j in range(1, args.batch)]
    mk = Megakernel((cfg, w), max_seq=PROMPT + GENERATE + 64, quant=args.quant, kv_dtype=args.kv_dtype, device=device,
                    batch=args.batch)
    sampler = ClockSampler(local) if rank == 0 else None
    kernel_ms, wall_s, launches, step_ns, clocks = measure(mk, args.batch, prompts, args, world, device, sampler)
    head = report(mk, args.batch, kernel_ms, wall_s, step_ns, args, world, device)
    single = None
    if args.batch > 1 and not args.no_batch1:
        mk.reset()
        k1, w1, l1, s1, _ = measure(mk, 1, prompts, args, world, device)
        single = report(mk, 1, k1, w1, s1, args, world, device)
        launches += l1

    # configuration 1 of the benchmark definition beside it: bf16 weights, batch 1, 32-token prompt, 128 greedy steps
    cfg1 = None
    if world == 1 and args.quant == "int8" and not args.no_cfg1 and (PROMPT, GENERATE) == (512, 512):
        del mk
        torch.cuda.empty_cache()
        cfg1 = measure_cfg1(args, device)

    if rank != 0:
        return
    out = {
        "metric": METRIC, "value": head["value"], "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": args.quant if args.quant == "int8" else "bf16", "data": "synthetic",
        "config": dict(workload_config(args.quant, args.batch, args.kv_dtype, cfg.vocab, cfg.n_layers),
                       median_decode_step_us=head["median_decode_step_us"],
                       bytes_per_decode_step=head["bytes_per_decode_step"]),
        "clocks": clocks,
        "e2e": head["e2e"],
        "gpu_launches": launches,
        "roofline": head["roofline"],
    }
    if single:
        out["batch1"] = {"value": single["value"], "unit": "tok/s", "ms_per_step": single["ms_per_step"],
                         "median_decode_step_us": single["median_decode_step_us"],
                         "bytes_per_decode_step": single["bytes_per_decode_step"], "e2e": single["e2e"],
                         "roofline": single["roofline"]}
    if cfg1:
        out["cfg1_bf16"] = cfg1
    if world == 1:
        # the library's own read-bandwidth probes on this GPU, beside the driver-measured peak the fractions use
        from megakernels_b200 import bw
        out["roofline"]["bw_probe_gbs"] = {m: round(bw.measure(m, gib=2.0, reps=3, device=device), 1) for m in bw.MODES}
    if world == 1 and not args.no_cpu_baseline:
        n_prompt, n_decode = 32, 48
        rate = cpu_reference_rate(cfg, w, prompt, n_prompt, n_decode)[0]
        out["cpu_baseline"] = {"value": rate, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"{n_prompt}-token prompt then {n_decode} greedy steps of one sequence, "
                                         "full depth, int8-dequantised weights in fp32"}
    print(json.dumps(out))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
