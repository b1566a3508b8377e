"""Command line: replay a workload of token-id requests through the engine and report
latency and throughput, in the manner of the reference's benchmark client.

    python -m iitj_llm_coopt_b200.cli --model DIR --workload FILE.jsonl --request-rate 4 --out result.json
    python -m iitj_llm_coopt_b200.cli --model DIR --workload synthetic:256:16-4096:16-512 --out result.json

Options keep the reference's names and meanings where it has them: the client's
--workload, --request-rate (default inf: all at once), --arrivals {rate,file}, --time-scale,
--max-concurrency, --limit, --seed, --out (bench/run.py:262-274) and the server's --model,
--max-num-seqs (256), --max-num-batched-tokens (2048), --kv-gb, --max-model-len (32768),
--gpu-memory-utilization (0.9), --dtype (engine/server.py:173-201).  There is no HTTP: the
requests go straight into the engine, in this process.  A workload file holds one JSON
object per line with `prompt_token_ids` and `max_tokens` (and optionally `id`, `category`,
`arrival_s`), as the reference's data files do (bench/run.py:26-30, 65-67); "synthetic:
N:PMIN-PMAX:OMIN-OMAX" draws N requests with uniform prompt and output lengths and
uniform-random token ids.  The summary has the reference's keys (bench/run.py:177-222):
num_requests, completed, failed, duration_s, output_throughput_tok_s,
total_throughput_tok_s, request_throughput, goodput_req_s and {ttft,tpot,itl_chunk,e2e}_
{mean,p50,p90,p99}; requests are sent with ignore_eos as the reference's client does.
"""
from __future__ import annotations

import argparse
import json
import math
import random
import sys
import time
from pathlib import Path


def load_workload(spec: str, vocab: int, limit=None, seed=0) -> list:
    if spec.startswith("synthetic:"):
        _, n, plen, olen = spec.split(":")
        pmin, pmax = (int(x) for x in plen.split("-"))
        omin, omax = (int(x) for x in olen.split("-"))
        rng = random.Random(seed)
        reqs = []
        for i in range(int(n)):
            p = rng.randint(pmin, pmax)
            reqs.append({"id": f"syn-{i}", "category": "long" if p > 2048 else "short",
                         "prompt_token_ids": [rng.randrange(vocab) for _ in range(p)], "prompt_len": p,
                         "max_tokens": rng.randint(omin, omax)})
    else:
        with open(spec, encoding="utf-8") as f:
            reqs = [json.loads(line) for line in f if line.strip()]
        for i, r in enumerate(reqs):
            r.setdefault("id", f"req-{i}")
            r.setdefault("category", "short")
            r.setdefault("prompt_len", len(r["prompt_token_ids"]))
    return reqs[:limit] if limit else reqs


def schedule(reqs, request_rate, arrivals, time_scale, seed) -> list:
    """Arrival offset (seconds from start) of every request (bench/run.py:33-45)."""
    if arrivals == "file":
        return [r["arrival_s"] * time_scale for r in reqs]
    if math.isinf(request_rate):
        return [0.0] * len(reqs)
    rng = random.Random(seed)
    t, out = 0.0, []
    for _ in reqs:
        out.append(t)
        t += rng.expovariate(request_rate)
    return out


def pct(xs, q):
    xs = sorted(x for x in xs if not math.isnan(x))
    if not xs:
        return float("nan")
    k = (len(xs) - 1) * q / 100.0
    lo, hi = math.floor(k), math.ceil(k)
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def summarize(results, duration, slo) -> dict:
    ok = [r for r in results if not r["error"]]
    out_tok = sum(r["output_tokens"] for r in ok)
    in_tok = sum(r["prompt_len"] for r in ok)
    ttft = [r["ttft"] for r in ok]
    tpot = [(r["e2e"] - r["ttft"]) / (r["output_tokens"] - 1) for r in ok if r["output_tokens"] > 1]
    gaps = [g for r in ok for g in r["chunk_gaps"]]
    e2e = [r["e2e"] for r in ok]

    def meets(r):
        t = slo["ttft_long"] if r["category"] == "long" else slo["ttft_short"]
        return r["ttft"] <= t and (r["e2e"] - r["ttft"]) / max(r["output_tokens"] - 1, 1) <= slo["tpot"]

    s = {"num_requests": len(results), "completed": len(ok), "failed": len(results) - len(ok),
         "duration_s": duration, "output_throughput_tok_s": out_tok / duration,
         "total_throughput_tok_s": (in_tok + out_tok) / duration, "request_throughput": len(ok) / duration,
         "goodput_req_s": sum(meets(r) for r in ok) / duration, "slo": slo}
    for name, xs in (("ttft", ttft), ("tpot", tpot), ("itl_chunk", gaps), ("e2e", e2e)):
        s[f"{name}_mean"] = sum(xs) / len(xs) if xs else float("nan")
        for q in (50, 90, 99):
            s[f"{name}_p{q}"] = pct(xs, q)
    return s


def run_workload(engine, reqs, offsets, temperature=0.0, max_concurrency=None) -> dict:
    results = [{"id": r["id"], "category": r.get("category", "short"), "prompt_len": r["prompt_len"],
                "max_tokens": r["max_tokens"], "scheduled_s": o, "start_s": 0.0, "ttft": float("nan"),
                "e2e": float("nan"), "output_tokens": 0, "chunk_gaps": [], "error": ""}
               for r, o in zip(reqs, offsets)]
    order = sorted(range(len(reqs)), key=lambda i: offsets[i])
    nxt, live = 0, 0
    t0 = time.perf_counter()

    def submit(i):
        nonlocal live
        res = results[i]
        res["start_s"] = time.perf_counter() - t0
        last = [None]

        def on_output(seq, new, done, res=res, last=last):
            nonlocal live
            now = time.perf_counter() - t0
            if new:
                if last[0] is None:
                    res["ttft"] = now - res["start_s"]
                else:
                    res["chunk_gaps"].append(round(now - last[0], 5))
                last[0] = now
                res["output_tokens"] += len(new)
            if done:
                res["e2e"] = now - res["start_s"]
                if seq.finish_reason == "out_of_pages":
                    res["error"] = "out_of_pages"
                live -= 1
        try:
            engine.new_sequence(reqs[i]["prompt_token_ids"], reqs[i]["max_tokens"], temperature, True, None, on_output)
            live += 1
        except ValueError as e:                    # e.g. a prompt longer than max_model_len
            res["error"] = str(e)[:300]

    while nxt < len(order) or engine.has_work():
        now = time.perf_counter() - t0
        while nxt < len(order) and offsets[order[nxt]] <= now and (not max_concurrency or live < max_concurrency):
            submit(order[nxt])
            nxt += 1
        if engine.has_work():
            engine.step()
        elif nxt < len(order):
            time.sleep(max(0.0, min(0.01, offsets[order[nxt]] - (time.perf_counter() - t0))))
    duration = time.perf_counter() - t0
    return {"results": results, "duration": duration}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and safetensors weights")
    ap.add_argument("--workload", required=True, help="JSONL file of requests, or synthetic:N:PMIN-PMAX:OMIN-OMAX")
    ap.add_argument("--request-rate", type=float, default=math.inf)
    ap.add_argument("--arrivals", choices=["rate", "file"], default="rate")
    ap.add_argument("--time-scale", type=float, default=1.0)
    ap.add_argument("--max-concurrency", type=int)
    ap.add_argument("--limit", type=int)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--kv-gb", type=float, default=None)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-model-len", type=int, default=32768)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--dtype", default="bfloat16", help="bfloat16 or float32")
    args = ap.parse_args(argv)

    from . import EngineConfig, build_engine
    ec = EngineConfig(dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages, kv_gb=args.kv_gb,
                      gpu_memory_utilization=args.gpu_memory_utilization, max_model_len=args.max_model_len,
                      max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens, seed=args.seed)
    engine = build_engine(args.model, ec)
    print(f"[engine] KV capacity {engine.kv_capacity_tokens} tokens ({engine.cache.num_pages} pages), "
          f"policy={engine.policy.name}", flush=True)
    reqs = load_workload(args.workload, engine.model_spec.vocab, args.limit, args.seed)
    offsets = schedule(reqs, args.request_rate, args.arrivals, args.time_scale, args.seed)
    run = run_workload(engine, reqs, offsets, args.temperature, args.max_concurrency)
    slo = {"ttft_short": 1.0, "ttft_long": 10.0, "tpot": 0.10}
    res = {"summary": summarize(run["results"], run["duration"], slo), "server_counters": dict(engine.counters),
           "requests": run["results"], "args": vars(args)}
    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    Path(args.out).write_text(json.dumps(res, indent=1, default=str))
    s = res["summary"]
    print(f"{args.workload}: {s['completed']}/{s['num_requests']} ok | out {s['output_throughput_tok_s']:.1f} tok/s | "
          f"TTFT p99 {s['ttft_p99']:.3f}s | TPOT p99 {s['tpot_p99'] * 1e3:.1f}ms | goodput {s['goodput_req_s']:.2f} req/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
