"""Trace replay (the program behind bin/trace_run).

It owns no forward pass, cache or loader: it builds the same engine that `LLM` builds
(`build_engine`), then drives `engine.runner.step` and the cache manager directly, without
the scheduler and without sampling.  The cache pool is sized for `--max-tokens` tokens
(rounded up to whole pages), so pages of finished requests are handed out again.

The reference has no such program; the nearest things are its teacher-forced scoring and
"prefill then append 1/2/5 tokens" checks (tests/m4_correctness.py:108-124,
tests/graph_check.py:31-49).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-requests", type=int, default=16, help="most requests live at a time")
    ap.add_argument("--device", default="cuda:0")
    return ap.parse_args(argv)


def run(args, lines, out=sys.stdout, kernels=None) -> int:
    import torch

    from . import EngineConfig, build_engine
    from .engine import StepEntry

    os.makedirs(args.out, exist_ok=True)
    pages = max(1, -(-args.max_tokens // args.page_size))
    ec = EngineConfig(dtype=args.dtype, page_size=args.page_size, num_pages=pages, max_num_seqs=args.max_requests,
                      max_num_batched_tokens=max(args.max_tokens, 1), max_model_len=1 << 30, device=args.device,
                      cuda_graphs=False)
    engine = build_engine(args.model, ec, kernels=kernels)
    runner, cache = engine.runner, engine.cache
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if not cache.has(rid):
                cache.admit(rid)
            entries.append(StepEntry(rid, [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        logits = runner.step(entries) if entries else None
        if logits is not None and logits.shape[0] > 0:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        elif args.device.startswith("cuda"):
            torch.cuda.synchronize()
        for rid in rec.get("end", []):
            if cache.has(rid):
                cache.release(rid)
        print(f"done {step}", file=out, flush=True)
    return 0


def main(argv=None) -> int:
    args = parse_args(argv)
    return run(args, sys.stdin)
