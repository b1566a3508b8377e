"""The command line's workload handling and summary on the CPU (fake engine), and a run on the GPU."""
import json
import math
import os
import subprocess
import sys

import pytest

from iitj_llm_coopt_b200 import cli
from test_scheduler import expected, make, prompt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_synthetic_workload_and_schedule():
    reqs = cli.load_workload("synthetic:20:4-30:2-9", vocab=97, seed=3)
    assert len(reqs) == 20 and all(4 <= r["prompt_len"] <= 30 and 2 <= r["max_tokens"] <= 9 for r in reqs)
    assert all(0 <= t < 97 for r in reqs for t in r["prompt_token_ids"])
    assert cli.schedule(reqs, math.inf, "rate", 1.0, 0) == [0.0] * 20
    offs = cli.schedule(reqs, 50.0, "rate", 1.0, 0)
    assert offs[0] == 0.0 and offs == sorted(offs) and offs == cli.schedule(reqs, 50.0, "rate", 1.0, 0)


def test_workload_file_and_summary_keys(tmp_path):
    path = tmp_path / "w.jsonl"
    rows = [{"id": f"q{i}", "category": "short", "prompt_token_ids": prompt(i, 5 + i), "max_tokens": 4,
             "arrival_s": 0.001 * i} for i in range(6)]
    path.write_text("\n".join(json.dumps(r) for r in rows))
    reqs = cli.load_workload(str(path), vocab=97, limit=5)
    assert len(reqs) == 5 and reqs[2]["prompt_len"] == 7
    eng, _, cache = make(pages=64, page=4, budget=16)
    run = cli.run_workload(eng, reqs, cli.schedule(reqs, math.inf, "file", 1.0, 0))
    s = cli.summarize(run["results"], run["duration"], {"ttft_short": 1.0, "ttft_long": 10.0, "tpot": 0.1})
    for key in ("num_requests", "completed", "failed", "duration_s", "output_throughput_tok_s", "total_throughput_tok_s",
                "request_throughput", "goodput_req_s", "ttft_mean", "ttft_p50", "ttft_p90", "ttft_p99", "tpot_p99",
                "itl_chunk_p50", "e2e_p99"):
        assert key in s
    assert s["completed"] == 5 and s["failed"] == 0
    assert all(r["output_tokens"] == 4 and len(r["chunk_gaps"]) == 3 for r in run["results"])
    assert cache.num_free == 64


@pytest.mark.gpu
def test_cli_runs_a_synthetic_workload(model_dirs, tmp_path):
    out = tmp_path / "res.json"
    proc = subprocess.run([sys.executable, "-m", "iitj_llm_coopt_b200.cli", "--model", model_dirs["C"], "--workload",
                           "synthetic:12:4-200:3-20", "--out", str(out), "--num-pages", "64", "--max-num-seqs", "4",
                           "--max-num-batched-tokens", "64"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(out.read_text())
    assert res["summary"]["completed"] == 12 and res["summary"]["failed"] == 0
    assert res["server_counters"]["request_success_total"] == 12
    assert "tok/s" in proc.stdout
