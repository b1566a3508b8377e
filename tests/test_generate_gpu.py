"""Greedy generation through the Python entry point and the command line, and the replay
program run as a user would run it, against the plain implementation."""
import json
import os
import struct
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as plain
import replay_cases as cases
from configs import CONFIGS
from iitj_llm_coopt_b200 import LLM, SamplingParams
from iitj_llm_coopt_b200.weights import write_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lively_dirs(tmp_path_factory):
    """The tiny models with a larger weight scale, so that greedy continuations vary."""
    out = {}
    for name, (cfg, seed, _page) in CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"lively_{name}"))
        write_model_dir(cfg, d, seed, std=0.08)
        out[name] = d
    return out


PROMPT_LENS = {"A": [5, 17, 33], "B": [1, 9, 40, 64, 130], "C": [3, 50, 90], "D": [2, 70], "E": [11, 60]}


def margins_ok(cfg, w, prompt, got, min_margin):
    """True if `got` equals the plain greedy continuation, allowing a different token only where the
    plain implementation's top two logits are closer than min_margin (then stop comparing)."""
    toks = list(prompt)
    for t in got:
        logits = plain.forward(cfg, w, toks)[-1]
        top = logits.topk(2)
        if t != int(top.indices[0]):
            return float(top.values[0] - top.values[1]) < min_margin and t == int(top.indices[1])
        toks.append(t)
    return True


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_generation_through_the_entry_point(lively_dirs, dtype, name):
    cfg_d, seed, page = CONFIGS[name]
    cfg, w = plain.read_model_dir(lively_dirs[name], torch.float32)
    prompts = list(cases.requests_for(cfg_d["vocab_size"], PROMPT_LENS[name], seed + 30).values())
    n_new = 16 if name == "A" else 24
    for budget, pages in ((2048, 256), (16, 40)):                 # roomy, then tight: portions and preemption
        llm = LLM(lively_dirs[name], dtype=dtype, page_size=page, num_pages=pages, max_num_seqs=4,
                  max_num_batched_tokens=budget)
        outs = llm.generate(prompts, SamplingParams(max_tokens=n_new, ignore_eos=True))
        for p, o in zip(prompts, outs):
            assert o.finish_reason == "length" and len(o.token_ids) == n_new
            if dtype == "float32":
                assert o.token_ids == plain.greedy_generate(cfg, w, p, n_new), (name, budget)
            else:
                assert margins_ok(cfg, w, p, o.token_ids, 0.05), (name, budget)
        llm.engine.cache.check()
        assert llm.engine.cache.num_free == pages
        del llm


def test_temperature_is_reproducible_per_request_and_mixes_with_greedy(lively_dirs):
    cfg_d, seed, page = CONFIGS["B"]
    prompts = list(cases.requests_for(cfg_d["vocab_size"], PROMPT_LENS["B"], seed + 31).values())
    params = [SamplingParams(max_tokens=24, temperature=0.8 if i % 2 == 0 else 0.0, ignore_eos=True, seed=100 + i)
              for i in range(len(prompts))]
    runs = []
    for budget, pages, seqs in ((2048, 256, 8), (24, 64, 2)):
        llm = LLM(lively_dirs["B"], dtype="float32", page_size=page, num_pages=pages, max_num_seqs=seqs,
                  max_num_batched_tokens=budget, seed=5)
        runs.append([o.token_ids for o in llm.generate(prompts, params)])
        del llm
    assert runs[0] == runs[1]                                     # same seeds, other batching: same tokens
    cfg, w = plain.read_model_dir(lively_dirs["B"], torch.float32)
    for i, p in enumerate(prompts):
        if i % 2 == 1:
            assert runs[0][i] == plain.greedy_generate(cfg, w, p, 24)
    llm = LLM(lively_dirs["B"], dtype="float32", page_size=page, num_pages=256, seed=6)
    other = [o.token_ids for o in llm.generate(prompts, params)]
    assert other[0] != runs[0][0]                                 # another engine seed, another draw


def test_eos_stops_generation(lively_dirs):
    cfg_d, seed, page = CONFIGS["C"]
    cfg, w = plain.read_model_dir(lively_dirs["C"], torch.float32)
    prompt = cases.requests_for(cfg_d["vocab_size"], [20], 77)["r0"]
    full = plain.greedy_generate(cfg, w, prompt, 12)
    import shutil, tempfile
    d = tempfile.mkdtemp()
    try:
        shutil.copy(os.path.join(lively_dirs["C"], "model.safetensors"), d)
        raw = json.load(open(os.path.join(lively_dirs["C"], "config.json")))
        raw["eos_token_id"] = full[4]
        json.dump(raw, open(os.path.join(d, "config.json"), "w"))
        llm = LLM(d, dtype="float32", num_pages=32)
        out = llm.generate([prompt], SamplingParams(max_tokens=12))[0]
        assert out.finish_reason == "stop" and out.token_ids == full[:full.index(full[4]) + 1]
    finally:
        shutil.rmtree(d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_program(model_dirs, tmp_path, dtype, name):
    """bin/trace_run as a subprocess: mixed trace over a pool sized by --max-tokens."""
    cfg_d, seed, page = CONFIGS[name]
    reqs = cases.requests_for(cfg_d["vocab_size"], [40, 75, 33, 130, 64, 20], seed + 40)
    steps, peak = cases.mixed(reqs, live=4, seed=3)
    lines = cases.as_jsonl(steps)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs[name],
                           "--dtype", dtype, "--out", str(out), "--max-tokens", str(peak), "--page-size", str(page)],
                          input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    cfg, w = plain.read_model_dir(model_dirs[name], torch.float32)
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    consumed = {rid: 0 for rid in reqs}
    worst = 0.0
    V = cfg_d["vocab_size"]
    for i, (entries, _ends) in enumerate(steps):
        wanted = sum(len(want) for _, _, want in entries)
        data = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(wanted, V)
        r = 0
        for rid, toks, want in entries:
            for wpos in want:
                want_row = ref[rid][consumed[rid] + wpos].numpy()
                worst = max(worst, float(np.abs(data[r] - want_row).max() / np.abs(want_row).max()))
                r += 1
            consumed[rid] += len(toks)
    assert worst <= (1e-4 if dtype == "float32" else 2e-2), worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_recomputes_the_same_tokens(lively_dirs, dtype):
    """A pool so small that running requests are preempted and re-prefilled with what they had generated:
    the tokens must be those of an engine with room for everything."""
    cfg_d, seed, page = CONFIGS["B"]
    prompts = list(cases.requests_for(cfg_d["vocab_size"], [30, 41, 25, 36], seed + 50).values())
    params = SamplingParams(max_tokens=40, ignore_eos=True)
    roomy = LLM(lively_dirs["B"], dtype=dtype, page_size=page, num_pages=200, max_num_seqs=4)
    want = [o.token_ids for o in roomy.generate(prompts, params)]
    assert roomy.engine.counters["num_preemptions_total"] == 0
    del roomy
    tight = LLM(lively_dirs["B"], dtype=dtype, page_size=page, num_pages=26, max_num_seqs=4, max_num_batched_tokens=48)
    outs = tight.generate(prompts, params)
    assert tight.engine.counters["num_preemptions_total"] >= 1 and max(o.num_preemptions for o in outs) >= 1
    got = [o.token_ids for o in outs]
    if dtype == "float32":
        assert got == want
    else:
        cfg, w = plain.read_model_dir(lively_dirs["B"], torch.float32)
        assert all(margins_ok(cfg, w, p, g, 0.05) for p, g in zip(prompts, got))
    tight.engine.cache.check()
    assert tight.engine.cache.num_free == 26


def test_wide_layer_at_the_benchmark_widths(tmp_path):
    """One layer with the widths of the benchmark model (hidden 4096, 32 heads / 8 kv heads of 128, inner 14336),
    a smaller vocabulary: float32 and bfloat16 against the plain implementation, whole and in portions."""
    cfg_d = {"architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 1,
             "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 2000, "rms_norm_eps": 1e-5,
             "rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
             "tie_word_embeddings": False, "max_position_embeddings": 131072}
    d = str(tmp_path / "wide")
    write_model_dir(cfg_d, d, seed=9)
    cfg, w = plain.read_model_dir(d, torch.float32)
    reqs = cases.requests_for(2000, [300, 140], 60)
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    from helpers import make_engine, rel_err, run_steps
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 2e-2)):
        eng = make_engine(d, dtype, 16, 64, max_num_seqs=2, max_num_batched_tokens=512)
        for steps in (cases.whole(reqs), cases.portions(reqs, [130, 2, 64, 1, 100])):
            rows = run_steps(eng, steps)
            for rid, toks in reqs.items():
                got = torch.stack([rows[(rid, i)] for i in range(len(toks))])
                assert rel_err(got, ref[rid]) <= tol, (dtype, rid)
        del eng


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "bfloat16"), ("D", "bfloat16")])
def test_many_random_requests_under_pressure(lively_dirs, name, dtype):
    """Forty requests of random lengths through a small pool and a small token budget: portions, mixed steps,
    captured decode steps of changing batch size, preemptions.  Every output against the plain implementation."""
    import random
    cfg_d, seed, page = CONFIGS[name]
    rng = random.Random(1234 + seed)
    prompts = [[rng.randrange(cfg_d["vocab_size"]) for _ in range(rng.choice([1, 2, 3, 7, 16, 17, 40, 90, 150]))]
               for _ in range(40)]
    params = [SamplingParams(max_tokens=rng.randint(1, 30), ignore_eos=True) for _ in prompts]
    pages = -(-(150 + 30) // page) * 3 // 2       # room for one and a half of the longest requests; six may run
    llm = LLM(lively_dirs[name], dtype=dtype, page_size=page, num_pages=pages, max_num_seqs=6, max_num_batched_tokens=48)
    outs = llm.generate(prompts, params)
    cfg, w = plain.read_model_dir(lively_dirs[name], torch.float32)
    for p, sp, o in zip(prompts, params, outs):
        assert len(o.token_ids) == sp.max_tokens and o.finish_reason == "length"
        if dtype == "float32":
            assert o.token_ids == plain.greedy_generate(cfg, w, p, sp.max_tokens)
        else:
            assert margins_ok(cfg, w, p, o.token_ids, 0.05)
    assert llm.engine.counters["num_preemptions_total"] >= 1
    assert llm.engine.runner.graph_replays > 0
    llm.engine.cache.check()
    assert llm.engine.cache.num_free == pages


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16")])
def test_padded_decode_batches(lively_dirs, name, dtype):
    """Thirteen requests that finish one after the other: their decode steps run at batch sizes 13 .. 9, which the
    step function pads to 16 with rows on the cache's padding page so that one captured graph serves them all.
    The padding rows must not show in anybody's output."""
    import random
    cfg_d, seed, page = CONFIGS[name]
    rng = random.Random(99 + seed)
    prompts = [[rng.randrange(cfg_d["vocab_size"]) for _ in range(rng.choice([3, 9, 20, 33]))] for _ in range(13)]
    params = [SamplingParams(max_tokens=12 + 3 * i, ignore_eos=True) for i in range(13)]
    llm = LLM(lively_dirs[name], dtype=dtype, page_size=page, num_pages=13 * (-(-(33 + 52) // page)) + 4, max_num_seqs=13,
              max_num_batched_tokens=512)
    outs = llm.generate(prompts, params)
    cfg, w = plain.read_model_dir(lively_dirs[name], torch.float32)
    for p, sp, o in zip(prompts, params, outs):
        assert len(o.token_ids) == sp.max_tokens
        if dtype == "float32":
            assert o.token_ids == plain.greedy_generate(cfg, w, p, sp.max_tokens)
        else:
            assert margins_ok(cfg, w, p, o.token_ids, 0.05)
    runner = llm.engine.runner
    assert runner.padded_steps > 0 and runner.graph_replays > 0


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16")])
def test_lookahead_changes_no_token(lively_dirs, name, dtype):
    """The same requests with and without launching steps ahead: greedy and temperature rows, a request that stops
    at an end-of-sequence token among others that go on, a tight pool and a roomy one.  Token for token the same."""
    import random, shutil, tempfile
    cfg_d, seed, page = CONFIGS[name]
    rng = random.Random(77 + seed)
    prompts = [[rng.randrange(cfg_d["vocab_size"]) for _ in range(rng.choice([1, 3, 9, 30, 64, 100]))] for _ in range(14)]
    params = [SamplingParams(max_tokens=rng.randint(1, 24), temperature=0.7 if i % 3 == 0 else 0.0, seed=300 + i)
              for i in range(len(prompts))]
    d = tempfile.mkdtemp()
    try:
        shutil.copy(os.path.join(lively_dirs[name], "model.safetensors"), d)
        raw = json.load(open(os.path.join(lively_dirs[name], "config.json")))
        # an end-of-sequence id that greedy decoding of the first prompts meets early
        probe = LLM(lively_dirs[name], dtype=dtype, page_size=page, num_pages=128, lookahead=False)
        first = probe.generate(prompts[:4], SamplingParams(max_tokens=12, ignore_eos=True))
        raw["eos_token_id"] = first[1].token_ids[5]
        del probe
        json.dump(raw, open(os.path.join(d, "config.json"), "w"))
        runs = {}
        for ahead in (False, True):
            for pages, budget, seqs in ((128, 512, 8), (-(-130 // page) * 2, 24, 3)):
                llm = LLM(d, dtype=dtype, page_size=page, num_pages=pages, max_num_seqs=seqs, max_num_batched_tokens=budget,
                          seed=9, lookahead=ahead)
                outs = llm.generate(prompts, params)
                runs[(ahead, pages)] = [(o.token_ids, o.finish_reason) for o in outs]
                assert llm.engine.lookahead == ahead
                llm.engine.cache.check()
                assert llm.engine.cache.num_free == pages
                del llm
        keys = list(runs)
        if dtype == "float32":
            assert all(runs[k] == runs[keys[0]] for k in keys)
        else:
            # bfloat16: another schedule means other batch sizes, other k-splits and other rounding, so a near-tie may
            # fall the other way; greedy rows must follow the plain implementation wherever its margin is clear
            cfg, w = plain.read_model_dir(lively_dirs[name], torch.float32)
            for k in keys:
                for i, (p, sp) in enumerate(zip(prompts, params)):
                    if sp.temperature == 0.0:
                        assert margins_ok(cfg, w, p, runs[k][i][0], 0.05), (k, i)
        assert any(reason == "stop" for _, reason in runs[keys[0]])
    finally:
        shutil.rmtree(d)


def test_captured_decode_steps_follow_a_context_that_outgrows_their_bounds(tmp_path):
    """Decoding from 450 to 1100 tokens of context with captured graphs on tiny D (head size 128): the split choice of
    the decode attention is frozen in a graph by an upper bound of the context (steps of 512 tokens), so the graph has
    to be captured anew when the context passes 512 and 1024, with several key splits and their merge inside the
    graph from then on.  The queries of this model are scaled up so that attention is peaked: keys left out by a
    stale split would move the logits.  Every decoded position is compared with the plain implementation and with
    the same engine without graphs."""
    from safetensors.torch import load_file, save_file
    from helpers import make_engine, rel_err, run_steps
    cfg_d, seed, page = CONFIGS["D"]
    d = str(tmp_path / "peaked")
    write_model_dir(cfg_d, d, seed)
    tensors = load_file(os.path.join(d, "model.safetensors"))
    for name in tensors:
        if name.endswith("q_proj.weight"):
            tensors[name] = (tensors[name].float() * 12.0).to(tensors[name].dtype)
    save_file(tensors, os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    total, head = 1100, 450
    reqs = cases.requests_for(cfg_d["vocab_size"], [total], seed + 70)
    cfg, w = plain.read_model_dir(d, torch.float32)
    ref = plain.forward(cfg, w, reqs["r0"])
    steps = cases.last_one_by_one(reqs, tail=total - head)
    rows = {}
    for graphs in (True, False):
        eng = make_engine(d, "bfloat16", page, -(-total // page) + 2, max_num_seqs=2, cuda_graphs=graphs)
        rows[graphs] = run_steps(eng, steps)
        if graphs:
            runner = eng.runner
            assert runner.graph_captures >= 3 and runner.graph_replays > 500      # bounds 512, 1024 and 1536
        del eng
    got = torch.stack([rows[True][("r0", i)] for i in range(total)])
    eager = torch.stack([rows[False][("r0", i)] for i in range(total)])
    assert rel_err(got, ref) <= 2e-2
    assert rel_err(got[head:], eager[head:]) <= 5e-3          # same kernels, the splits chosen from a bound: rounding only
