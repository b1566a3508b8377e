"""The index arrays that the step function hands to the model (positions, token-to-request map, cache slots, block
tables, logits rows) against a per-request restatement from the cache manager's own lists, over random sequences of
steps: portions of changing size beside single tokens, requests that end and whose slots and pages are used again,
a group with a window that gives pages back.  Host logic only (CPU, plain-torch kernel double)."""
import random

import pytest
import torch

from iitj_llm_coopt_b200 import EngineConfig, build_engine
from iitj_llm_coopt_b200.engine import StepEntry
from torch_kernels import TorchKernels

from test_toy_parts import ToyWindowArch, ToyWindowConfig


def check_arrays(ctx, entries, starts, cache):
    T = sum(len(e.tokens) for e in entries)
    assert ctx.num_tokens == T and ctx.num_requests == len(entries)
    want_ids, want_pos, want_req, want_rows, cu = [], [], [], [], [0]
    for b, (e, s) in enumerate(zip(entries, starts)):
        want_ids += e.tokens
        want_pos += list(range(s, s + len(e.tokens)))
        want_req += [b] * len(e.tokens)
        want_rows += [cu[-1] + w for w in e.want]
        cu.append(cu[-1] + len(e.tokens))
    assert ctx.token_ids.tolist() == want_ids and ctx.positions.tolist() == want_pos
    assert ctx.token_request.tolist() == want_req and ctx.cu_seqlens.tolist() == cu
    assert ctx.seq_lens.tolist() == [s + len(e.tokens) for e, s in zip(entries, starts)]
    assert ctx.logit_rows.tolist() == want_rows
    assert ctx.state_slots.tolist() == [cache.state_slot(e.request) for e in entries]
    assert ctx.first_portion.tolist() == [1 if s == 0 else 0 for s in starts]
    for g in cache.paged:
        meta = ctx.group(g)
        slots = [x for e, s in zip(entries, starts) for x in cache.slots(g, e.request, s, s + len(e.tokens))]
        assert meta.slots.tolist() == slots
        table = meta.block_table.tolist()
        for b, e in enumerate(entries):
            pages = [max(p, 0) for p in cache.table(g, e.request)]
            assert table[b][:len(pages)] == pages and not any(table[b][len(pages):])


@pytest.mark.parametrize("window", [0, 10])
@pytest.mark.parametrize("seed", range(5))
def test_step_arrays_follow_the_cache_tables(seed, window):
    rng = random.Random(seed)
    ec = EngineConfig(dtype="float32", page_size=4, num_pages=60, max_num_seqs=4, device="cpu")
    eng = build_engine(None, ec, config=ToyWindowConfig(16, window), architecture=ToyWindowArch(), random_seed=1,
                       kernels=TorchKernels())
    runner, cache = eng.runner, eng.cache
    assert cache.windowed == (window > 0)
    seen = {}

    real_forward = runner.model.forward

    def spy(ctx):
        seen["ctx"] = ctx
        return real_forward(ctx)
    runner.model.forward = spy
    live, next_id = {}, 0
    for _ in range(60):
        while len(live) < 4 and rng.random() < 0.6:
            live[f"q{next_id}"] = rng.randint(1, 70)         # tokens the request will bring in all
            cache.admit(f"q{next_id}")
            next_id += 1
        if not live:
            continue
        entries, starts = [], []
        for rid in rng.sample(sorted(live), rng.randint(1, len(live))):
            left = live[rid] - cache.num_tokens(rid)
            n = min(left, rng.choice([1, 1, 2, 3, 7, 16]))
            toks = [rng.randrange(200) for _ in range(n)]
            entries.append(StepEntry(rid, toks, sorted(rng.sample(range(n), rng.randint(0, min(n, 2))))))
            starts.append(cache.num_tokens(rid))
        runner.step(entries)
        # (the tables are read after the step: where a window gave pages back meanwhile they read -1, while the step's
        #  own arrays were built before, when those pages were still held)
        if cache.windowed:
            check_arrays_windowed(seen["ctx"], entries, starts, cache)
        else:
            check_arrays(seen["ctx"], entries, starts, cache)
        cache.check()
        for e in entries:
            if cache.num_tokens(e.request) == live[e.request]:
                cache.release(e.request)
                del live[e.request]
    for rid in list(live):
        cache.release(rid)
    cache.check()
    assert cache.num_free == 60


def check_arrays_windowed(ctx, entries, starts, cache):
    """As check_arrays, for a cache with a windowed group: pages that the step itself let go (after its arrays were
    built) read -1 in the tables now; the arrays must hold the page that was there, which no other request got since."""
    T = sum(len(e.tokens) for e in entries)
    assert ctx.num_tokens == T
    assert ctx.positions.tolist() == [p for e, s in zip(entries, starts) for p in range(s, s + len(e.tokens))]
    assert ctx.token_request.tolist() == [b for b, e in enumerate(entries) for _ in e.tokens]
    ps = cache.page_size
    for g in cache.paged:
        meta = ctx.group(g)
        table, slots, row = meta.block_table.tolist(), meta.slots.tolist(), 0
        for b, (e, s) in enumerate(zip(entries, starts)):
            pages = cache.table(g, e.request)
            for lp, p in enumerate(pages):
                assert table[b][lp] == p or p == -1
            assert not any(table[b][len(pages):])
            for pos in range(s, s + len(e.tokens)):
                assert slots[row] == table[b][pos // ps] * ps + pos % ps and table[b][pos // ps] >= 0
                row += 1
