#!/usr/bin/env python3
"""Headline benchmark: decode tokens/s and prefill tokens/s of the Llama 3.1 8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers L]

Prints ONE JSON line.  `value` is decoded tokens per second at the given batch (default 8)
with `context` tokens per request already in the cache, timed on the device with one pair
of CUDA events around the K decode steps (model step + sampling kernel, run back to back:
each step takes its tokens on the device from the ids the step before sampled).  `e2e` is
the same metric through the engine's public entry point (host token ids in, host token ids
out every step; the prompts' prefill and W warm-up decode steps run first, then the rate is
counted over the timed decode steps).  `prefill` is one 2,048-token prompt in one step; `roofline`
relates the decode step's mandatory HBM reads to its time; `points` holds decode at batch
1 and 64.  Weights are random (seeded, drawn on the device), token ids are random.

`--impl reference` times the unmodified reference engine (a copy of its tree under
`baseline/_ref`) on the same metric and configuration: see baseline/reference_arm.py.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from iitj_llm_coopt_b200.presets import SHAPES      # config.json dicts of the benchmark shapes (data only; imports no kernels)

BENCH_SHAPES = ("8b", "3b", "1b", "toy")            # the default line is the 8B shape; the others are for sweeps and trials
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            peaks = {k: float(raw[k]) for k in FALLBACK_PEAKS if k in raw}
            if "hbm_gbs" in peaks and "bf16_tflops" in peaks:
                peaks.setdefault("bf16_tflops_sustained", peaks["bf16_tflops"])
                return peaks, "measured"
        except (OSError, ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background for the whole run: SM clock and throttle reasons.  `busy()` brackets the
    timed phases; the median clock is taken over the samples that fell inside them, the throttle reasons over all."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines, self.windows = None, [], []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def busy(self):
        sampler = self

        class _Window:
            def __enter__(self):
                self.t0 = time.perf_counter()

            def __exit__(self, *exc):
                sampler.windows.append((self.t0, time.perf_counter()))
                return False
        return _Window()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm_all, sm_busy, mx, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for stamp, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm_all.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            # a sample describes the 100 ms before it arrived
            if any(t0 <= stamp <= t1 + 0.1 for t0, t1 in self.windows):
                sm_busy.append(sm_all[-1])
            for name, flag in zip(names, parts[3:7]):
                if flag == "Active":
                    reasons.add(name)
        under = sm_busy or sm_all
        return {"sm_mhz": statistics.median(under) if under else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm_all), "samples_under_load": len(sm_busy), "reasons": sorted(reasons)}


def matmul_weight_bytes(cfg, itemsize=2):
    """Bytes of every matrix a decode step reads once: the layers' four projections and the head."""
    h, inter, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    H, Hkv, D, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    per_layer = (H + 2 * Hkv) * D * h + h * H * D + 2 * inter * h + h * inter
    return (L * per_layer + V * h) * itemsize


def prefill_flops(cfg, T, rows=1):
    h, inter, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    H, Hkv, D, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    linear = 2 * T * ((H + 2 * Hkv) * D * h + h * H * D + 2 * inter * h + h * inter)
    attention = 4 * (T * (T + 1) // 2) * H * D
    return L * (linear + attention) + 2 * rows * h * V


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (reported)")
    ap.add_argument("--shape", choices=BENCH_SHAPES, default="8b", help="layer sizes: Llama 3.1 8B (the benchmark), 3.2 3B or 3.2 1B")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one phase alone with few repetitions and print a short line (for profilers)")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step by itself (for profiling)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (only --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.only:
        args.no_points = args.no_e2e = True

    peaks, peak_source = load_peaks()
    model_name, shape_cfg = SHAPES[args.shape]
    cfg = dict(shape_cfg)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    B, C, K, W = args.batch, args.context, args.steps, args.warmup
    weight_bytes = matmul_weight_bytes(cfg)
    p_flops = prefill_flops(cfg, args.prefill_tokens)

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
        try:
            line = reference_arm.run(cfg, model_name, full_layers, B, C, K, W, args.prefill_tokens, not args.no_points,
                                     not args.no_e2e, not args.no_prefill, peaks, peak_source, ClockSampler(), weight_bytes,
                                     p_flops)
        except Exception as e:          # the reference's own code failed on this box: say so, as one line
            line = {"impl": "reference", "unavailable": f"the reference engine raised {type(e).__name__}: {str(e)[:300]}"}
        print(json.dumps(line))
        return 0

    import torch

    from iitj_llm_coopt_b200 import LLM, LlamaConfig, SamplingParams, StepEntry

    typed = LlamaConfig.from_dict(cfg)
    page = 16
    biggest = max(B, 1 if args.no_points else 64)
    # a step shape is captured into a CUDA graph at its fourth sighting: those sightings come before the W warm-up steps
    PRIME = 0 if args.no_graphs else 5
    pool_tokens = biggest * (C + max(K, 96) + W + PRIME + 2 * page) + args.prefill_tokens + 4 * page
    t_build = time.time()
    # the engine is built by the public entry point; the device-timed phases drive its step function directly
    llm = LLM(config=typed, random_seed=2, dtype="bfloat16", page_size=page, num_pages=-(-pool_tokens // page),
              max_num_seqs=max(biggest, 8),
              # the end-to-end phase prefills its B prompts in one step, so that all B requests decode together from
              # the first decode step to the last (with a smaller budget they would start, and end, one after the other)
              max_num_batched_tokens=max(args.prefill_tokens, biggest, 0 if args.no_e2e else B * C),
              max_model_len=C + max(K, 96) + W + PRIME + 64, seed=0, cuda_graphs=not args.no_graphs)
    engine = llm.engine
    runner, cache, sampler, kernels = engine.runner, engine.cache, engine.sampler, engine.sampler.k
    for g in cache.groups:                      # contexts "already in the cache": random keys and values
        if g.storage is not None:
            g.storage.normal_(0.0, 0.5)
    torch.cuda.synchronize()
    build_s = time.time() - t_build
    gen = torch.Generator().manual_seed(0)

    def decode_run(batch, steps, warmup):
        """Device-timed decode steps at `batch` with C tokens per request in the cache."""
        ids = [f"d{batch}_{i}" for i in range(batch)]
        for r in ids:
            cache.admit(r)
            cache.ensure(r, C)
            cache.advance(r, C)
        toks = torch.randint(0, typed.vocab_size, (batch,), generator=gen).tolist()
        # Steps run back to back as in serving: each step's input tokens are the ids the sampling kernel of the
        # step before left on the device (no host round trip in between); one pair of events brackets the timed
        # steps, with a synchronize on both sides.
        prev = None
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches = 0
        for it in range(-PRIME, warmup + steps):
            if it == warmup:
                torch.cuda.synchronize()
                launches = kernels.launches
                start.record()
            if prev is None:
                entries = [StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]
            else:
                entries = [StepEntry(r, [0], [0], source_rows=[i]) for i, r in enumerate(ids)]
            logits = runner.step(entries, prev_ids=prev)
            out, _ = sampler._buffers(batch)
            kernels.sample(logits, None, None, out)
            prev = out
        end.record()
        torch.cuda.synchronize()
        times = [start.elapsed_time(end) / steps] * steps
        launches = kernels.launches - launches
        for r in ids:
            cache.release(r)
        return times, launches

    def prefill_run(T, reps, warmup):
        times = []
        for it in range(warmup + reps):
            cache.admit("p")
            toks = torch.randint(0, typed.vocab_size, (T,), generator=gen).tolist()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            runner.step([StepEntry("p", toks, [T - 1])])
            end.record()
            torch.cuda.synchronize()
            cache.release("p")
            if it >= warmup:
                times.append(start.elapsed_time(end))
        return times

    if args.only == "prefill":
        t = sorted(prefill_run(args.prefill_tokens, max(1, K), 1))
        print(json.dumps({"only": "prefill", "tokens": args.prefill_tokens, "ms": t[len(t) // 2], "min_ms": t[0], "reps": len(t)}))
        return 0
    if args.only == "decode":
        t, n = decode_run(B, max(1, K), W)
        print(json.dumps({"only": "decode", "batch": B, "ms": sum(t) / len(t), "launches_per_step": n / len(t)}))
        return 0
    clocks = ClockSampler()
    clocks.start()              # sampled over every timed phase of the run: decode, prefill, points, end to end
    with clocks.busy():
        times, launches = decode_run(B, K, W)
    ms = sum(times) / len(times)
    value = B / (ms / 1e3)

    kv_bytes = B * (C + PRIME + W + K / 2) * typed.kv_bytes_per_token(2)
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9

    with clocks.busy():
        p_times = prefill_run(args.prefill_tokens, 5, 3) if not args.no_prefill else [float("nan")]
    p_ms = statistics.median(p_times)
    prefill = {"value": args.prefill_tokens / (p_ms / 1e3), "tokens": args.prefill_tokens, "ms": p_ms,
               "frac": p_flops / (p_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), "peak": f"of {peak_source}"}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            with clocks.busy():
                t, _ = decode_run(b, max(8, K // 2), W)
            points[f"decode_b{b}"] = b / (sum(t) / len(t) / 1e3)

    e2e = None
    if not args.no_e2e:
        # through the public entry point: host token ids in (prompts), host token ids out (every step's tokens reach
        # the callback).  The prompts are prefilled in one step; then come untimed decode steps (the eager sightings
        # of the step's shape, its capture into a graph, and the clocks' recovery from the prefill at full power,
        # which the first dozen decode steps still show), then the timed ones.
        prompts = [torch.randint(0, typed.vocab_size, (C,), generator=gen).tolist() for _ in range(B)]
        stamps = []

        def on_out(seq, new, fin):
            stamps.append(time.perf_counter())

        WE, KE = max(W, 24), max(K, 64)
        with clocks.busy():
            llm.generate(prompts, SamplingParams(max_tokens=WE + KE + 1, ignore_eos=True), on_output=on_out)
            torch.cuda.synchronize()
        # every decode step hands one token of each request to the callback: the timed region runs from the
        # last callback of warm-up step WE to the last callback of all (KE steps of B tokens)
        per_step = sorted(stamps)
        t_start, t_last = per_step[B * (WE + 1) - 1], per_step[-1]
        decoded = len(per_step) - B * (WE + 1)
        h2d = runner.copied_bytes        # the last decode step's index arrays (ids, positions, slots, block tables): one copy
        e2e = {"value": decoded / (t_last - t_start), "unit": "tok/s", "steps": decoded // B, "warmup": WE,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B}

    clock_rec = clocks.stop()
    kernels.check_health()          # raises if any kernel gave up on a bounded wait during the run
    line = {
        "metric": f"decode tok/s at batch {B} ({model_name[:-13]} shape, {C}-token contexts); prefill and batch 1/64 alongside",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": model_name, "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": B, "seq_len": C, "page_size": page, "parallelism": "single-gpu",
                   "l2": f"inputs larger than L2 (a step reads {weight_bytes / 1e9:.1f} GB of weights)", "weights": "random seed 2"},
        "clocks": clock_rec,
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peak_source": f"of {peak_source}"},
        "points": points,
        "graph_priming_steps": PRIME,
        "health": "ok",
        "build_seconds": build_s,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
