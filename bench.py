"""Decode throughput of the megakernel on the benchmark's int8 0.8B configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (configuration 2 of the benchmark definition): the 0.8B Gated-DeltaNet / attention hybrid,
vocab 151936, int8 per-channel weights quantised from seeded N(0, 0.02) bf16 weights, batch 1, a
512-token uniform-random prompt already in the recurrent state and KV cache, then 512 greedy decode
steps.  One bench "step" is one such 512-token generation: one kernel launch.  Synthetic weights and
prompt stand in for the checkpoint and text the reference measures on.

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

METRIC = "decode tok/s at batch 1 (0.8B hybrid, int8 per-channel, 512-token prompt + 512 greedy steps)"
PROMPT, GENERATE = 512, 512
L2_BYTES = 126e6
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch, per generated token, from the
# ncu capture summarised in profiles/decode_kernel_int8_64prompt_16steps.md (a 16-step launch at a 64-token
# context, scaled by steps; the KV part grows with context, the weight part does not).
NCU_DRAM_BYTES_PER_TOKEN = (10.533937e9 + 337.758208e6) / 16


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


def bytes_per_token(mk):
    """Algorithmic bytes one decode step must move: every weight once, the DeltaNet state read and
    written, the KV cache read at the average context of the generation."""
    body, head = mk.weight_bytes
    kv = mk.kv_bytes_per_pos() * (PROMPT + GENERATE // 2)
    return body + head + mk.state_bytes() + kv


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
        "config": {"workload": "qwen3.5-0.8b hybrid, int8-dequantised weights, batch 1", "prompt": PROMPT,
                   "generate": GENERATE, "vocab": cfg.vocab, "layers": cfg.n_layers},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    global PROMPT, GENERATE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--quant", default="int8", choices=["int8", "bf16"])
    ap.add_argument("--kv-dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="shrink the case (profiling only)")
    ap.add_argument("--generate", type=int, default=GENERATE, help="shrink the case (profiling only)")
    args = ap.parse_args()
    PROMPT, GENERATE = args.prompt, args.generate
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode megakernel has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    from megakernels_b200.engine import Megakernel
    cfg, w, prompt = build_model(args.quant)
    mk = Megakernel((cfg, w), max_seq=PROMPT + GENERATE + 64, quant=args.quant, kv_dtype=args.kv_dtype, device=device)
    last = mk.prefill(prompt)                 # the prompt goes through the kernel, one token per step
    snap = mk.snapshot()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()

    def one_step(timing=False):
        mk.restore(snap)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        ids = mk.run([last], n_generate=GENERATE, timing=timing)
        e1.record(stream)
        return ids, e0, e1

    for _ in range(args.warmup):
        ids, _, _ = one_step()
    assert len(ids) == GENERATE
    # ---- timed region: kernel time with inputs resident (CUDA events on the launching stream)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    launches0 = mk.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    start.record(stream)
    kernel_events, step_ns = [], []
    for _ in range(args.steps):
        ids, e0, e1 = one_step(timing=True)
        kernel_events.append((e0, e1))
        step_ns += mk.last_step_ns
    end.record(stream)
    barrier()
    wall_s = time.perf_counter() - wall0
    launches = mk.launches - launches0
    clocks = sampler.stop() if rank == 0 else None
    kernel_ms = [a.elapsed_time(b) for a, b in kernel_events]      # launch + readback of one generation
    local_ms = sum(kernel_ms)
    tokens = args.steps * GENERATE
    total_ms, total_tokens = aggregate(local_ms, tokens, world, device)
    value = total_tokens / (total_ms / 1e3)
    # e2e: the public call with host inputs and outputs, wall clock around the same K steps
    e2e_ms, _ = aggregate(wall_s * 1e3, tokens, world, device)
    e2e = total_tokens / (e2e_ms / 1e3)

    if rank != 0:
        return
    peak, peak_kind = measured_peak_gbs()
    bpt = bytes_per_token(mk)
    launch_s = statistics.mean(kernel_ms) / 1e3
    achieved = bpt * GENERATE / launch_s / 1e9
    median_step_us = statistics.median(step_ns) / 1e3
    out = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": args.quant if args.quant == "int8" else "bf16", "data": "synthetic",
        "config": {"workload": "qwen3.5-0.8b hybrid (24 layers, hidden 1024, vocab 151936), "
                               f"{args.quant} weights, batch 1, replicas only",
                   "prompt_tokens": PROMPT, "decode_steps_per_bench_step": GENERATE, "kv_dtype": args.kv_dtype,
                   "l2": "weights streamed per decode step (0.65 GB int8) exceed the 126 MB L2; no flush needed",
                   "median_decode_step_us": median_step_us, "bytes_per_token": bpt},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4 + 4, "d2h_bytes_per_step": 8 * GENERATE + 32 + 4},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8TBs": achieved / 8000.0,
                     "traffic": NCU_DRAM_BYTES_PER_TOKEN * GENERATE if NCU_DRAM_BYTES_PER_TOKEN else None,
                     "algorithmic_bytes_per_launch": bpt * GENERATE},
    }
    if world == 1 and not args.no_cpu_baseline:
        n_prompt, n_decode = 32, 48
        rate = cpu_reference_rate(cfg, w, prompt, n_prompt, n_decode)[0]
        out["cpu_baseline"] = {"value": rate, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"{n_prompt}-token prompt then {n_decode} greedy steps, full depth, "
                                         "int8-dequantised weights in fp32"}
    print(json.dumps(out))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
