"""Command line: run a workload of token-id requests through the engine, in this process, and report
latency, throughput and (on request) the generated token ids, in the manner of the reference's benchmark client.

    python -m iitj_llm_coopt_b200.cli --model DIR --workload FILE.jsonl --request-rate 4 --out result.json
    python -m iitj_llm_coopt_b200.cli --shape tinyA --random-seed 0 --workload synthetic:12:4-200:3-20 --save-tokens --out r.json
    python -m iitj_llm_coopt_b200.cli --workload baseline:1b-continuous --out out_1b.json
    python -m iitj_llm_coopt_b200.cli --workload baseline:3b-mixed --out out_3b.json

Options keep the reference's names and meanings where it has them: the client's --workload, --request-rate
(default inf: all at once), --arrivals {rate,file}, --time-scale, --max-concurrency, --limit, --seed, --out
(bench/run.py:262-274) and the server's --model, --max-num-seqs (256), --max-num-batched-tokens (2048), --kv-gb,
--max-model-len (32768), --gpu-memory-utilization (0.9), --dtype (engine/server.py:173-201).  There is no HTTP: the
requests go straight into the engine.  In place of a model folder, `--shape NAME --random-seed S` builds a model of
a named shape (presets.py) with random weights.

Workloads:
  FILE.jsonl                       one JSON object per line with `prompt_token_ids` and `max_tokens` (optionally `id`,
                                   `category`, `arrival_s`), as the reference's data files (bench/run.py:26-30, 65-67)
  synthetic:N:PMIN-PMAX:OMIN-OMAX  N requests, prompt and output lengths uniform in the ranges, uniform-random ids
  baseline:1b-continuous           256 requests, prompts uniform in [16, 4096], outputs uniform in [16, 512], seed 3,
                                   on the Llama 3.2 1B shape, all sent at once (continuous batching)
  baseline:3b-mixed                32 requests that decode 400 tokens from 64-token prompts beside six 16,384-token
                                   prompts fed in 512-token portions (token budget 544), seed 4, Llama 3.2 3B shape
A baseline workload brings its shape, seed and token budget with it; options given on the command line win.

The result file has the reference's layout (bench/run.py:248-253, 177-222): `summary` with num_requests, completed,
failed, duration_s, output_throughput_tok_s, total_throughput_tok_s, request_throughput, goodput_req_s, slo and
{ttft,tpot,itl_chunk,e2e}_{mean,p50,p90,p99}; `server_counters`; `requests` (one record each: id, category,
prompt_len, max_tokens, scheduled_s, start_s, ttft, e2e, output_tokens, chunk_gaps, error, and with --save-tokens
`token_ids`); `args`.  Requests are sent with ignore_eos, as the reference's client sends them.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

SLO = {"ttft_short": 1.0, "ttft_long": 10.0, "tpot": 0.10}      # seconds (bench/run.py:227)

# The two serving workloads of the benchmark's smaller shapes: shape, seed, engine options, and how the requests are drawn.
BASELINE_WORKLOADS = {
    "1b-continuous": {"shape": "1b", "seed": 3, "max_num_batched_tokens": 2048,
                      "groups": [{"count": 256, "prompt": (16, 4096), "output": (16, 512)}]},
    "3b-mixed": {"shape": "3b", "seed": 4, "max_num_batched_tokens": 544,
                 "groups": [{"count": 32, "prompt": (64, 64), "output": (400, 400)},
                            {"count": 6, "prompt": (16384, 16384), "output": (32, 32)}]},
}


# ---- workloads -------------------------------------------------------------------------------
def _drawn_requests(groups, vocab: int, seed: int, prefix: str) -> list:
    """Requests of each group in turn: lengths uniform in the group's ranges (ends included), uniform-random ids."""
    rng = np.random.default_rng(seed)
    reqs = []
    for g in groups:
        plens = rng.integers(g["prompt"][0], g["prompt"][1] + 1, size=g["count"])
        olens = rng.integers(g["output"][0], g["output"][1] + 1, size=g["count"])
        for p, o in zip(plens.tolist(), olens.tolist()):
            reqs.append({"id": f"{prefix}-{len(reqs)}", "category": "long" if p > 2048 else "short",
                         "prompt_token_ids": rng.integers(0, vocab, size=p).tolist(), "prompt_len": p, "max_tokens": o})
    return reqs


def load_workload(spec: str, vocab: int, limit=None, seed=0) -> list:
    """The requests of workload `spec` (see the module text) as dicts with id, category, prompt_token_ids,
    prompt_len, max_tokens (and arrival_s where a file gives it)."""
    if spec.startswith("baseline:"):
        name = spec.split(":", 1)[1]
        if name not in BASELINE_WORKLOADS:
            raise ValueError(f"baseline workload {name!r} is not known; known: {', '.join(sorted(BASELINE_WORKLOADS))}")
        reqs = _drawn_requests(BASELINE_WORKLOADS[name]["groups"], vocab, seed, name)
    elif spec.startswith("synthetic:"):
        try:
            _, n, plen, olen = spec.split(":")
            prompt = tuple(int(x) for x in plen.split("-"))
            output = tuple(int(x) for x in olen.split("-"))
            groups = [{"count": int(n), "prompt": prompt, "output": output}]
            assert len(prompt) == 2 and len(output) == 2
        except (ValueError, AssertionError):
            raise ValueError(f"workload {spec!r}: want synthetic:N:PMIN-PMAX:OMIN-OMAX") from None
        reqs = _drawn_requests(groups, vocab, seed, "syn")
    else:
        with open(spec, encoding="utf-8") as f:
            reqs = [json.loads(line) for line in f if line.strip()]
        for i, r in enumerate(reqs):
            r.setdefault("id", f"req-{i}")
            r.setdefault("category", "short")
            r.setdefault("prompt_len", len(r["prompt_token_ids"]))
    return reqs[:limit] if limit else reqs


def arrival_offsets(reqs, request_rate: float, arrivals: str, time_scale: float, seed: int) -> list:
    """Seconds from the start at which each request is sent: the file's `arrival_s` scaled by `time_scale`
    (arrivals == "file"), all at once (an infinite rate), or a Poisson process of `request_rate` requests a second
    that starts with the first request at 0 (the meanings of bench/run.py:33-45)."""
    if arrivals == "file":
        return [float(r["arrival_s"]) * time_scale for r in reqs]
    if not reqs or math.isinf(request_rate):
        return [0.0] * len(reqs)
    gaps = np.random.default_rng(seed).exponential(1.0 / request_rate, size=len(reqs))
    gaps[0] = 0.0
    return np.cumsum(gaps).tolist()


# ---- per-request records and the summary -------------------------------------------------------
@dataclass
class RequestRecord:
    """What the client side knows of one request.  Times are seconds; `arrivals` are the moments (from the start of
    the run) at which tokens of this request reached the caller."""
    id: str
    category: str
    prompt_len: int
    max_tokens: int
    scheduled_s: float
    start_s: float = 0.0
    arrivals: list = field(default_factory=list)
    output_tokens: int = 0
    token_ids: list | None = None           # kept only when asked for
    finished_s: float = math.nan
    error: str = ""

    def note(self, now: float, new_tokens: list, done: bool, failure: str = "") -> None:
        if new_tokens:
            self.arrivals.append(now)
            self.output_tokens += len(new_tokens)
            if self.token_ids is not None:
                self.token_ids.extend(new_tokens)
        if done:
            self.finished_s = now
            self.error = failure

    @property
    def ttft(self) -> float:
        return self.arrivals[0] - self.start_s if self.arrivals else math.nan

    @property
    def e2e(self) -> float:
        return self.finished_s - self.start_s

    @property
    def tpot(self) -> float:
        """Seconds per token after the first (nan for a single token)."""
        return (self.e2e - self.ttft) / (self.output_tokens - 1) if self.output_tokens > 1 else math.nan

    @property
    def chunk_gaps(self) -> list:
        return np.round(np.diff(self.arrivals), 5).tolist() if len(self.arrivals) > 1 else []

    def meets(self, slo: dict) -> bool:
        first = slo["ttft_long"] if self.category == "long" else slo["ttft_short"]
        per_token = 0.0 if math.isnan(self.tpot) else self.tpot
        return self.ttft <= first and per_token <= slo["tpot"]

    def as_dict(self) -> dict:
        d = {"id": self.id, "category": self.category, "prompt_len": self.prompt_len, "max_tokens": self.max_tokens,
             "scheduled_s": self.scheduled_s, "start_s": self.start_s, "ttft": self.ttft, "e2e": self.e2e,
             "output_tokens": self.output_tokens, "chunk_gaps": self.chunk_gaps, "error": self.error}
        if self.token_ids is not None:
            d["token_ids"] = self.token_ids
        return d


def _spread(prefix: str, values) -> dict:
    """mean, p50, p90, p99 of the values that are numbers (nan everywhere if there are none)."""
    xs = np.asarray([v for v in values if not math.isnan(v)], dtype=np.float64)
    if xs.size == 0:
        return {f"{prefix}_{k}": math.nan for k in ("mean", "p50", "p90", "p99")}
    p50, p90, p99 = np.percentile(xs, [50, 90, 99])
    return {f"{prefix}_mean": float(xs.mean()), f"{prefix}_p50": float(p50), f"{prefix}_p90": float(p90),
            f"{prefix}_p99": float(p99)}


def summarize(records: list, duration: float, slo: dict) -> dict:
    """The run's summary under the reference's key names (bench/run.py:177-222)."""
    good = [r for r in records if not r.error]
    generated = sum(r.output_tokens for r in good)
    prompted = sum(r.prompt_len for r in good)
    summary = {
        "num_requests": len(records), "completed": len(good), "failed": len(records) - len(good),
        "duration_s": duration,
        "output_throughput_tok_s": generated / duration,
        "total_throughput_tok_s": (prompted + generated) / duration,
        "request_throughput": len(good) / duration,
        "goodput_req_s": sum(1 for r in good if r.meets(slo)) / duration,
        "slo": slo,
    }
    summary.update(_spread("ttft", [r.ttft for r in good]))
    summary.update(_spread("tpot", [r.tpot for r in good]))
    summary.update(_spread("itl_chunk", [g for r in good for g in r.chunk_gaps]))
    summary.update(_spread("e2e", [r.e2e for r in good]))
    return summary


# ---- the run ---------------------------------------------------------------------------------
def run_workload(engine, reqs, offsets, temperature=0.0, max_concurrency=None, save_tokens=False) -> dict:
    """Sends every request at its offset (at most `max_concurrency` in flight), steps the engine until all are
    done; returns {"records": [RequestRecord], "duration": seconds}."""
    records = [RequestRecord(r["id"], r.get("category", "short"), r["prompt_len"], r["max_tokens"], float(o),
                             token_ids=[] if save_tokens else None) for r, o in zip(reqs, offsets)]
    pending = sorted(range(len(reqs)), key=lambda i: offsets[i])[::-1]     # a stack: the next one to send is last
    in_flight = 0
    t0 = time.perf_counter()

    def send(i):
        nonlocal in_flight
        rec = records[i]
        rec.start_s = time.perf_counter() - t0

        def on_output(seq, new, done, rec=rec):
            nonlocal in_flight
            failure = "out_of_pages" if done and seq.finish_reason == "out_of_pages" else ""
            rec.note(time.perf_counter() - t0, new, done, failure)
            if done:
                in_flight -= 1
        try:
            engine.new_sequence(reqs[i]["prompt_token_ids"], reqs[i]["max_tokens"], temperature, True, None, on_output)
            in_flight += 1
        except ValueError as e:                    # e.g. a prompt longer than max_model_len
            rec.note(rec.start_s, [], True, str(e)[:300])

    while pending or engine.has_work():
        now = time.perf_counter() - t0
        while pending and offsets[pending[-1]] <= now and (not max_concurrency or in_flight < max_concurrency):
            send(pending.pop())
        if engine.has_work():
            engine.step()
        elif pending:
            time.sleep(max(0.0, min(0.01, offsets[pending[-1]] - (time.perf_counter() - t0))))
    return {"records": records, "duration": time.perf_counter() - t0}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", help="folder with config.json and safetensors weights")
    ap.add_argument("--shape", help="in place of --model: a named shape with random weights (8b, 3b, 1b, tinyA, tinyB)")
    ap.add_argument("--random-seed", type=int, default=None, help="seed of the random weights of --shape")
    ap.add_argument("--workload", required=True,
                    help="JSONL file of requests, synthetic:N:PMIN-PMAX:OMIN-OMAX, baseline:1b-continuous or baseline:3b-mixed")
    ap.add_argument("--request-rate", type=float, default=math.inf)
    ap.add_argument("--arrivals", choices=["rate", "file"], default="rate")
    ap.add_argument("--time-scale", type=float, default=1.0)
    ap.add_argument("--max-concurrency", type=int)
    ap.add_argument("--limit", type=int)
    ap.add_argument("--seed", type=int, default=None, help="seed of the workload's lengths, ids and arrivals (default 0)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--save-tokens", action="store_true", help="keep every request's generated token ids in the result file")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=None, help="token budget of a step (default 2048)")
    ap.add_argument("--kv-gb", type=float, default=None)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-model-len", type=int, default=32768)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--dtype", default="bfloat16", help="bfloat16 or float32")
    args = ap.parse_args(argv)

    # a baseline workload brings its shape, seed and token budget; what the command line gives wins
    if args.workload.startswith("baseline:"):
        preset = BASELINE_WORKLOADS.get(args.workload.split(":", 1)[1])
        if preset is None:
            ap.error(f"unknown baseline workload; known: {', '.join(sorted(BASELINE_WORKLOADS))}")
        if args.model is None and args.shape is None:
            args.shape = preset["shape"]
        if args.seed is None:
            args.seed = preset["seed"]
        if args.max_num_batched_tokens is None:
            args.max_num_batched_tokens = preset["max_num_batched_tokens"]
        if args.random_seed is None:
            args.random_seed = preset["seed"]
    if args.seed is None:
        args.seed = 0
    if args.max_num_batched_tokens is None:
        args.max_num_batched_tokens = 2048
    if (args.model is None) == (args.shape is None):
        ap.error("give either --model DIR or --shape NAME")

    from . import EngineConfig, build_engine
    ec = EngineConfig(dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages, kv_gb=args.kv_gb,
                      gpu_memory_utilization=args.gpu_memory_utilization, max_model_len=args.max_model_len,
                      max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens, seed=args.seed)
    if args.model is not None:
        engine = build_engine(args.model, ec)
    else:
        from .config.registry import architecture_for
        from .presets import shape_config
        raw = shape_config(args.shape)
        engine = build_engine(None, ec, config=architecture_for(raw).config_class.from_dict(raw),
                              random_seed=args.random_seed or 0)
    print(f"[engine] KV capacity {engine.kv_capacity_tokens} tokens ({engine.cache.num_pages} pages), "
          f"policy={engine.policy.name}", flush=True)
    reqs = load_workload(args.workload, engine.model_spec.vocab, args.limit, args.seed)
    offsets = arrival_offsets(reqs, args.request_rate, args.arrivals, args.time_scale, args.seed)
    run = run_workload(engine, reqs, offsets, args.temperature, args.max_concurrency, args.save_tokens)
    check = getattr(engine.sampler.k, "check_health", None)
    if check is not None:
        check()
    res = {"summary": summarize(run["records"], run["duration"], dict(SLO)), "server_counters": dict(engine.counters),
           "requests": [r.as_dict() for r in run["records"]], "args": vars(args)}
    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    Path(args.out).write_text(json.dumps(res, indent=1, default=str))
    s = res["summary"]
    print(f"{args.workload}: {s['completed']}/{s['num_requests']} ok in {s['duration_s']:.2f} s | "
          f"out {s['output_throughput_tok_s']:.1f} tok/s | total {s['total_throughput_tok_s']:.1f} tok/s | "
          f"TTFT p99 {s['ttft_p99']:.3f}s | TPOT p50 {s['tpot_p50'] * 1e3:.1f}ms p99 {s['tpot_p99'] * 1e3:.1f}ms | "
          f"goodput {s['goodput_req_s']:.2f} req/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
