"""The command line's workload handling and summary on the CPU (fake engine), and runs on the GPU: the generated
token ids it hands out against the plain implementation, a named shape with random weights, and the engine's
three ways of sizing its key/value pool."""
import json
import math
import os
import subprocess
import sys

import pytest

from iitj_llm_coopt_b200 import cli
from test_scheduler import expected, make, prompt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_synthetic_workload_and_arrivals():
    reqs = cli.load_workload("synthetic:20:4-30:2-9", vocab=97, seed=3)
    assert len(reqs) == 20 and all(4 <= r["prompt_len"] <= 30 and 2 <= r["max_tokens"] <= 9 for r in reqs)
    assert all(len(r["prompt_token_ids"]) == r["prompt_len"] for r in reqs)
    assert all(0 <= t < 97 for r in reqs for t in r["prompt_token_ids"])
    assert reqs == cli.load_workload("synthetic:20:4-30:2-9", vocab=97, seed=3)          # the seed decides
    assert reqs != cli.load_workload("synthetic:20:4-30:2-9", vocab=97, seed=4)
    assert cli.arrival_offsets(reqs, math.inf, "rate", 1.0, 0) == [0.0] * 20
    offs = cli.arrival_offsets(reqs, 50.0, "rate", 1.0, 0)
    assert offs[0] == 0.0 and offs == sorted(offs) and offs == cli.arrival_offsets(reqs, 50.0, "rate", 1.0, 0)
    assert 0.1 < offs[-1] < 1.5                                                          # 19 gaps of 20 ms on average
    with pytest.raises(ValueError):
        cli.load_workload("synthetic:20:4-30", vocab=97)


def test_baseline_workloads_are_the_benchmark_configurations():
    one = cli.load_workload("baseline:1b-continuous", vocab=128256, seed=3)
    assert len(one) == 256
    assert all(16 <= r["prompt_len"] <= 4096 and 16 <= r["max_tokens"] <= 512 for r in one)
    assert min(r["prompt_len"] for r in one) < 200 and max(r["prompt_len"] for r in one) > 3900
    mixed = cli.load_workload("baseline:3b-mixed", vocab=128256, seed=4)
    assert [r["prompt_len"] for r in mixed] == [64] * 32 + [16384] * 6
    assert [r["max_tokens"] for r in mixed] == [400] * 32 + [32] * 6
    assert [r["category"] for r in mixed] == ["short"] * 32 + ["long"] * 6
    assert cli.BASELINE_WORKLOADS["3b-mixed"]["max_num_batched_tokens"] == 512 + 32
    with pytest.raises(ValueError):
        cli.load_workload("baseline:nothing", vocab=10)


def test_workload_file_and_summary_keys(tmp_path):
    path = tmp_path / "w.jsonl"
    rows = [{"id": f"q{i}", "category": "short", "prompt_token_ids": prompt(i, 5 + i), "max_tokens": 4,
             "arrival_s": 0.001 * i} for i in range(6)]
    path.write_text("\n".join(json.dumps(r) for r in rows))
    reqs = cli.load_workload(str(path), vocab=97, limit=5)
    assert len(reqs) == 5 and reqs[2]["prompt_len"] == 7
    eng, _, cache = make(pages=64, page=4, budget=16)
    run = cli.run_workload(eng, reqs, cli.arrival_offsets(reqs, math.inf, "file", 1.0, 0), save_tokens=True)
    s = cli.summarize(run["records"], run["duration"], dict(cli.SLO))
    for key in ("num_requests", "completed", "failed", "duration_s", "output_throughput_tok_s", "total_throughput_tok_s",
                "request_throughput", "goodput_req_s", "slo", "ttft_mean", "ttft_p50", "ttft_p90", "ttft_p99", "tpot_mean",
                "tpot_p50", "tpot_p99", "itl_chunk_p50", "itl_chunk_p99", "e2e_mean", "e2e_p99"):
        assert key in s
    assert s["completed"] == 5 and s["failed"] == 0 and s["goodput_req_s"] > 0
    for r, rec in zip(reqs, run["records"]):
        d = rec.as_dict()
        assert d["output_tokens"] == 4 and len(d["chunk_gaps"]) == 3 and d["error"] == ""
        assert d["token_ids"] == expected(r["prompt_token_ids"], 4)       # the ids the (fake) model generates
        assert d["ttft"] > 0 and d["e2e"] >= d["ttft"]
    assert cache.num_free == 64


def test_summary_numbers():
    recs = []
    for i, (first, per_token, n) in enumerate([(0.5, 0.01, 11), (2.0, 0.02, 21), (0.2, 0.2, 2)]):
        r = cli.RequestRecord(f"r{i}", "short", 10, n, 0.0, start_s=1.0)
        for j in range(n):
            r.note(1.0 + first + per_token * j, [7], j == n - 1)
        recs.append(r)
    failed = cli.RequestRecord("bad", "short", 10, 5, 0.0)
    failed.note(0.0, [], True, "prompt too long")
    s = cli.summarize(recs + [failed], 10.0, dict(cli.SLO))
    assert s["num_requests"] == 4 and s["completed"] == 3 and s["failed"] == 1
    assert s["output_throughput_tok_s"] == pytest.approx(34 / 10.0)
    assert s["total_throughput_tok_s"] == pytest.approx(64 / 10.0)
    assert s["goodput_req_s"] == pytest.approx(1 / 10.0)       # the second misses the first-token limit, the third the per-token one
    assert s["ttft_p50"] == pytest.approx(0.5) and s["ttft_mean"] == pytest.approx(0.9)
    assert s["tpot_p50"] == pytest.approx(0.02) and s["tpot_p99"] == pytest.approx(0.2, rel=0.05)
    assert s["e2e_p50"] == pytest.approx(0.6)


@pytest.mark.gpu
def test_cli_hands_out_the_plain_implementations_tokens(model_dirs, tmp_path):
    """--save-tokens in float32 on tiny C: every request's ids equal greedy decoding by the plain implementation."""
    import torch
    import plain_llama as plain
    import replay_cases as cases
    from configs import CONFIGS
    cfg_d, seed, page = CONFIGS["C"]
    prompts = list(cases.requests_for(cfg_d["vocab_size"], [3, 40, 17, 90, 5, 64], seed + 60).values())
    work = tmp_path / "w.jsonl"
    work.write_text("\n".join(json.dumps({"id": f"p{i}", "prompt_token_ids": p, "max_tokens": 6 + i})
                              for i, p in enumerate(prompts)))
    out = tmp_path / "res.json"
    proc = subprocess.run([sys.executable, "-m", "iitj_llm_coopt_b200.cli", "--model", model_dirs["C"], "--workload", str(work),
                           "--out", str(out), "--num-pages", "64", "--max-num-seqs", "4", "--max-num-batched-tokens", "48",
                           "--dtype", "float32", "--save-tokens"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(out.read_text())
    assert res["summary"]["completed"] == len(prompts) and res["summary"]["failed"] == 0
    assert res["server_counters"]["request_success_total"] == len(prompts)
    cfg, w = plain.read_model_dir(model_dirs["C"], torch.float32)
    for i, (p, rec) in enumerate(zip(prompts, res["requests"])):
        assert rec["id"] == f"p{i}" and rec["output_tokens"] == 6 + i
        assert rec["token_ids"] == plain.greedy_generate(cfg, w, p, 6 + i), i
    assert "tok/s" in proc.stdout


@pytest.mark.gpu
def test_cli_runs_a_named_shape_with_random_weights(tmp_path):
    out = tmp_path / "res.json"
    proc = subprocess.run([sys.executable, "-m", "iitj_llm_coopt_b200.cli", "--shape", "tinyB", "--random-seed", "5", "--workload",
                           "synthetic:12:4-200:3-20", "--out", str(out), "--num-pages", "128", "--page-size", "8",
                           "--max-num-seqs", "4", "--max-num-batched-tokens", "64", "--save-tokens"],
                          cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(out.read_text())
    assert res["summary"]["completed"] == 12 and res["summary"]["failed"] == 0
    assert all(len(r["token_ids"]) == r["output_tokens"] == r["max_tokens"] for r in res["requests"])
    assert all(0 <= t < 320 for r in res["requests"] for t in r["token_ids"])


@pytest.mark.gpu
@pytest.mark.parametrize("how", ["kv_gb", "free_memory"])
def test_pool_sized_from_bytes_or_from_free_memory(model_dirs, how):
    """The two ways of sizing the key/value pool that no explicit page count takes: --kv-gb, and what is left of the
    GPU's memory (capped at what max_num_seqs requests of max_model_len tokens can fill).  The pool has the size the
    rule gives and generation is unchanged."""
    import torch
    import plain_llama as plain
    from configs import CONFIGS
    from iitj_llm_coopt_b200 import LLM, SamplingParams
    cfg_d, seed, page = CONFIGS["A"]
    per_page = 2 * cfg_d["num_hidden_layers"] * cfg_d["num_key_value_heads"] * cfg_d["head_dim"] * page * 4   # float32
    if how == "kv_gb":
        kv_gb = (300 + 1) * per_page / 2**30              # (the storage holds one padding page beyond the pool)
        llm = LLM(model_dirs["A"], dtype="float32", page_size=page, kv_gb=kv_gb, max_num_seqs=4)
        assert llm.engine.cache.num_pages == 300
    else:
        llm = LLM(model_dirs["A"], dtype="float32", page_size=page, max_num_seqs=4, max_model_len=200)
        assert llm.engine.cache.num_pages == 4 * math.ceil(200 / page)           # memory is plentiful: the cap decides
        free, total = torch.cuda.mem_get_info()
        assert llm.engine.cache.num_pages * per_page < 0.9 * total
    cfg, w = plain.read_model_dir(model_dirs["A"], torch.float32)
    p = [5, 9, 200, 31, 77]
    out = llm.generate([p], SamplingParams(max_tokens=8, ignore_eos=True))[0]
    assert out.token_ids == plain.greedy_generate(cfg, w, p, 8)
