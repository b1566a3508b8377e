"""The engine's step function against the plain implementation, for every way of cutting
the same requests into steps: whole; most in one step and the last 32 tokens one by one;
portions of changing size; and mixed batches over a pool so small that pages are used
again.  Runs on the GPU with the CUDA kernels in float32 and bfloat16 (`-m gpu`), and on
the CPU with the plain-torch kernel double, which checks the host logic alone."""
import pytest
import torch

import plain_llama as plain
import replay_cases as cases
from configs import CONFIGS
from helpers import make_engine, rel_err, run_steps

FP32_TOL, BF16_TOL = 1e-4, 2e-2
LENGTHS = {"A": [5, 17, 33, 70, 129], "B": [1, 9, 40, 64, 130], "C": [3, 66, 150, 31], "D": [2, 130, 47, 80], "E": [70, 3, 41]}

GPU = pytest.mark.gpu
CASES = [pytest.param("cpu", "float32", n, id=f"cpu-fp32-{n}") for n in "AB"] + \
        [pytest.param("cuda:0", dt, n, marks=GPU, id=f"gpu-{dt}-{n}")
         for dt in ("float32", "bfloat16") for n in "ABCDE"]


def reference_rows(model_dir, reqs):
    cfg, w = plain.read_model_dir(model_dir, torch.float32)
    return {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}


def compare(rows, ref, reqs, tol):
    worst = 0.0
    for rid, toks in reqs.items():
        got = torch.stack([rows[(rid, i)] for i in range(len(toks))])
        worst = max(worst, rel_err(got, ref[rid]))
    assert worst <= tol, worst
    return worst


@pytest.fixture(scope="module")
def refs(model_dirs):
    out = {}
    for name, lens in LENGTHS.items():
        cfg, seed, _ = CONFIGS[name]
        reqs = cases.requests_for(cfg["vocab_size"], lens, seed + 10)
        out[name] = (reqs, reference_rows(model_dirs[name], reqs))
    return out


@pytest.mark.parametrize("device,dtype,name", CASES)
def test_every_way_of_cutting(model_dirs, refs, device, dtype, name):
    reqs, ref = refs[name]
    page = CONFIGS[name][2]
    tol = FP32_TOL if dtype == "float32" else BF16_TOL
    mixed_steps, peak = cases.mixed(reqs, live=4, seed=1)
    pages = peak // page                      # just enough for the live requests: pages are used again
    eng = make_engine(model_dirs[name], dtype, page, pages, device=device, max_num_seqs=4)
    results = {}
    for label, steps in (("whole", cases.whole(reqs)), ("last32", cases.last_one_by_one(reqs)),
                         ("portions", cases.portions(reqs)), ("mixed", mixed_steps)):
        rows = run_steps(eng, steps)
        eng.cache.check()
        assert eng.cache.num_free == pages     # everything was given back
        results[label] = compare(rows, ref, reqs, tol)
    # the ways of cutting agree with each other far more closely than with the oracle's tolerance
    print(name, dtype, results)


@pytest.mark.parametrize("device,dtype,name", CASES)
def test_first_tokens_of_a_sequence(model_dirs, refs, device, dtype, name):
    """Positions 0, 1, 2 fed one token at a time, each its own step."""
    reqs, ref = refs[name]
    page = CONFIGS[name][2]
    rid, toks = next((r, t) for r, t in reqs.items() if len(t) >= 3)
    eng = make_engine(model_dirs[name], dtype, page, 8, device=device, max_num_seqs=2)
    rows = run_steps(eng, [([(rid, toks[i:i + 1], [0])], []) for i in range(3)])
    got = torch.stack([rows[(rid, i)] for i in range(3)])
    assert rel_err(got, ref[rid][:3]) <= (FP32_TOL if dtype == "float32" else BF16_TOL)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_long_decoding(model_dirs, dtype, name):
    """A 40-token prompt and then 360 (B) or 600 (C) tokens one by one; every position compared."""
    cfg, seed, page = CONFIGS[name]
    total = 400 if name == "B" else 640
    reqs = cases.requests_for(cfg["vocab_size"], [total], seed + 20)
    ref = reference_rows(model_dirs[name], reqs)
    eng = make_engine(model_dirs[name], dtype, page, -(-total // page) + 1, max_num_seqs=2)
    rows = run_steps(eng, cases.last_one_by_one(reqs, tail=total - 40))
    compare(rows, ref, reqs, FP32_TOL if dtype == "float32" else BF16_TOL)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_ways_of_cutting_agree_closely(model_dirs, refs, name):
    """In float32 the same position computed whole and in portions differs by rounding only."""
    reqs, _ = refs[name]
    page = CONFIGS[name][2]
    eng = make_engine(model_dirs[name], "float32", page, 64, max_num_seqs=4)
    a = run_steps(eng, cases.whole(reqs))
    b = run_steps(eng, cases.portions(reqs))
    worst = max(rel_err(b[k], a[k]) for k in a)
    assert worst < 1e-5, worst
