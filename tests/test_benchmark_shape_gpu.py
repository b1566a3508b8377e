"""The paths the benchmark times, compared with the plain implementation at the benchmark's own layer sizes:
Llama 3.1 8B widths (hidden 4096, 32 heads / 8 key-value heads of 128, inner 14336) with the real vocabulary of
128,256 tokens, untied, 2 of the 32 layers.  One prompt of 3,400 tokens is among the requests, so a whole-prompt
step runs the CTA-pair SwiGLU product (from 640 tokens), portions against its later context run the prefill
attention with its keys shared out over several CTAs (contexts from 3,072 tokens), its last tokens decode with
several key splits, and mixed steps run 512-token portions beside decoded tokens.

The oracle is tests/plain_llama.py in float32 on the GPU (the CPU would take minutes at these sizes), with TF32
switched off.  Teacher-forced logits at every position, as the reference scores them
(tests/m4_correctness.py:104-124), and "a prefix, then a few tokens appended" as tests/graph_check.py:31-49.
"""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_llama as plain
import replay_cases as cases
import torch_kernels as R
from iitj_llm_coopt_b200.engine import StepEntry
from iitj_llm_coopt_b200.weights import write_model_dir

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "max_position_embeddings": 131072, "eos_token_id": 128001,
}
LENGTHS = [3400, 700, 150, 40]
SIZES = [512, 2, 130, 700, 64, 7, 300, 33, 1024, 2]      # portions: below 128, 129..639, from 640 tokens, down to two
PAGE = 16


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    d = str(tmp_path_factory.mktemp("llama8b_widths_2_layers"))
    write_model_dir(WIDE, d, seed=11, device="cuda")
    cfg, w = plain.read_model_dir(d, torch.float32, device="cuda")
    reqs = cases.requests_for(WIDE["vocab_size"], LENGTHS, 70)
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    del w
    torch.cuda.empty_cache()
    return d, reqs, ref


def run_and_compare(engine, steps, reqs, ref):
    """Runs the trace and compares every wanted row with the oracle's row on the device; returns the largest
    error relative to the largest logit of the request.  Every position of every request must have been wanted."""
    runner, cache = engine.runner, engine.cache
    scale = {rid: ref[rid].abs().max() for rid in reqs}
    worst = torch.zeros((), device="cuda")
    seen = {rid: set() for rid in reqs}
    for entries, ends in steps:
        es = []
        for rid, toks, want in entries:
            if not cache.has(rid):
                cache.admit(rid)
            es.append(StepEntry(rid, list(toks), list(want)))
        starts = [cache.num_tokens(e.request) for e in es]
        logits = runner.step(es)
        r = 0
        for e, s in zip(es, starts):
            n = len(e.want)
            if n:
                pos = torch.tensor([s + w for w in e.want], device="cuda")
                err = (logits[r:r + n] - ref[e.request][pos]).abs().max() / scale[e.request]
                worst = torch.maximum(worst, err)
                seen[e.request].update(s + w for w in e.want)
                r += n
        for rid in ends:
            cache.release(rid)
    for rid, toks in reqs.items():
        assert seen[rid] == set(range(len(toks))), rid
    return worst.item()


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 2e-2)])
def test_llama8b_widths_2_of_32_layers_every_way_of_cutting(wide, dtype, tol):
    from helpers import make_engine
    d, reqs, ref = wide
    mixed_steps, peak = cases.mixed(reqs, live=4, seed=2, sizes=SIZES)
    pages = peak // PAGE                               # just enough for the live requests: pages are used again
    eng = make_engine(d, dtype, PAGE, pages, max_num_seqs=4, max_num_batched_tokens=4096)
    results = {}
    for label, steps in (("whole", cases.whole(reqs)), ("last32", cases.last_one_by_one(reqs)),
                         ("portions", cases.portions(reqs, SIZES)), ("mixed", mixed_steps)):
        results[label] = run_and_compare(eng, steps, reqs, ref)
        eng.cache.check()
        assert eng.cache.num_free == pages
    print(dtype, results)
    assert max(results.values()) <= tol, results
    k = eng.runner.model.k
    assert k.gemm_status() == 0 and k.gemm_pair_status() == 0 and k.attention_status() == 0
    if dtype == "bfloat16":
        assert eng.runner.graph_replays > 0            # the decoded tail ran from a captured graph


def _headline_case(lens, page, heads, kv_heads, head_dim, seed):
    """A paged cache for single-token queries at the ends of contexts `lens`; page ids shuffled."""
    need = [-(-n // page) for n in lens]
    total = sum(need) + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total, generator=g)
    table = torch.zeros(len(lens), max(need), dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        table[b, :n] = perm[at:at + n].to(torch.int32)
        at += n
    gd = torch.Generator(device="cuda").manual_seed(seed + 1)
    cache = (torch.randn((total, 2, kv_heads, page, head_dim), generator=gd, device="cuda") * 0.3).to(torch.bfloat16)
    meta = SimpleNamespace(block_table=table.cuda(), token_request=torch.arange(len(lens), dtype=torch.int32).cuda(),
                           positions=torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda(),
                           query_lens=[1] * len(lens), seq_lens_host=list(lens))
    return cache, meta


@pytest.mark.parametrize("bound", [None, "graph"])
@pytest.mark.parametrize("fused", [False, True])
def test_decode_attention_at_the_headline_shape(decode_loads, fused, bound):
    """Batch 64 of 32 heads / 8 key-value heads of 128, pages of 16, contexts of 8192 give or take a few and one of
    16,400, with either kernel (TMA boxes, or copies by the threads): the split chosen from the contexts themselves and,
    as a captured graph has it, from an upper bound.  In
    some requests one far key stands out (on the first and last key of a split and beside them), so that a
    split that is dropped, or merged with the wrong weight, changes the result from about 3 to about 0."""
    from iitj_llm_coopt_b200 import kernels
    from iitj_llm_coopt_b200.kernels import AttentionPlan, PartialSums
    K = kernels.load()
    heads, kv_heads, D, page = 32, 8, 128, 16
    lens = [8192 + d for d in (-3, -1, 0, 1, 2, 15, 16, 17)] * 8
    lens[5] = 16400
    cache, meta = _headline_case(lens, page, heads, kv_heads, D, 300)
    tokens, width = len(lens), (heads + 2 * kv_heads) * D
    plan = AttentionPlan(meta.query_lens, meta.seq_lens_host, "cuda", total_tokens=tokens)
    if bound == "graph":
        plan.context_bound = (max(plan.decode_pos) + 512) // 512 * 512
    meta.attention_plan = plan
    kps, splits = plan.split(kv_heads, 0, K.sm_count, D, plan.context_bound)
    assert splits > 1 and kps * splits >= max(lens)
    gq = torch.Generator(device="cuda").manual_seed(301)
    qkv = torch.randn((tokens, width), generator=gq, device="cuda") * 0.3
    # the planted keys: request b looks for a key at `far[b]`
    far = {0: 0, 1: kps - 1, 2: kps, 3: kps + 1, 4: 2 * kps - 1, 5: 2 * kps, 13: 3 * kps - 1, 6: lens[6] - 2, 7: 4097, 9: 63}
    far = {b: min(p, lens[b] - 2) for b, p in far.items()}        # (a split edge beyond a request's keys: its last key but one)
    direction = torch.randn(D, generator=gq, device="cuda")
    direction = direction / direction.norm()
    for b, pos in far.items():
        pg, off = int(meta.block_table[b, pos // page]), pos % page
        cache[pg, 0, :, off] = (direction * 40.0).to(torch.bfloat16)
        cache[pg, 1, :, off] = 3.0
        qkv[b, :heads * D] = (direction * 12.0).repeat(heads)
    pos = meta.positions.long()
    slots = (meta.block_table[torch.arange(tokens, device="cuda"), pos // page].long() * page + pos % page).to(torch.int32)
    meta.slots = slots
    out = torch.empty(tokens, heads * D, device="cuda", dtype=torch.bfloat16)
    if fused:
        # the qkv product as two partial sums, no rotation (cos 1, sin 0): the kernel adds, stores the token's key and
        # value, and attends
        parts = torch.stack([qkv * 0.5, qkv * 0.5]).contiguous()       # (halves add up exactly)
        cos = torch.ones(tokens, D // 2, device="cuda")
        sin = torch.zeros(tokens, D // 2, device="cuda")
        want_cache = cache.clone()
        q16 = qkv.to(torch.bfloat16)
        R.ref_store(want_cache, q16, slots, heads, kv_heads, D)
        ps = PartialSums(K, parts, torch.zeros(tokens, width, device="cuda", dtype=torch.bfloat16))
        assert K.can_fuse_decode(ps, meta, cache, heads, kv_heads, D)
        K.attention_decode_fused(ps, (cos, sin), slots, cache, meta, out, heads, kv_heads, D)
        want = R.ref_paged_attention(q16, want_cache, meta.block_table, meta.token_request, meta.positions, heads,
                                     kv_heads, D)
        assert torch.equal(cache, want_cache)
    else:
        q16 = qkv.to(torch.bfloat16)
        K.attention(q16, cache, meta, out, heads, kv_heads, D)
        want = R.ref_paged_attention(q16, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads, D)
    err = (out.float() - want).abs().max().item()
    assert err <= 1.6e-2 * want.abs().max().item(), err
    for b in far:
        assert (out[b].float() - 3.0).abs().max().item() < 0.1, b
