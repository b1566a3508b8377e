"""The scheduler's decisions and the engine's bookkeeping on the CPU, with a fake step
function whose "model" is a hash of the request's whole token history: the generated
tokens then depend on nothing but the prompt, so every schedule must produce them."""
import pytest

from iitj_llm_coopt_b200.cache import CacheManager
from iitj_llm_coopt_b200.config.specs import CacheNeed
from iitj_llm_coopt_b200.engine import Engine, Sequence, StaticPolicy

VOCAB = 97
NEED = CacheNeed(kind="paged_kv", kv_heads=1, head_dim=16)


def next_token(history):
    h = 7
    for t in history:
        h = (h * 31 + t + 1) % 1000003
    return h % VOCAB


def expected(prompt, n, eos=()):
    toks, out = list(prompt), []
    for _ in range(n):
        t = next_token(toks)
        toks.append(t)
        out.append(t)
        if t in eos:
            break
    return out


class FakeRunner:
    """Follows the step function's contract: feeds on top of what the cache holds."""

    def __init__(self, cache):
        self.cache, self.history, self.log = cache, {}, []

    def step(self, entries):
        rows = []
        self.log.append([(e.request, len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            start = self.cache.num_tokens(e.request)
            if start == 0:
                self.history[e.request] = []        # a new request, or one recomputed after a preemption
            hist = self.history.setdefault(e.request, [])
            assert len(hist) == start, "tokens must continue where the cache ends"
            self.cache.ensure(e.request, start + len(e.tokens))
            for i, t in enumerate(e.tokens):
                hist.append(t)
                if i in e.want:
                    rows.append(next_token(hist))
            self.cache.advance(e.request, start + len(e.tokens))
        return rows


class FakeSampler:
    def sample(self, logits, rows):
        assert len(logits) == len(rows)
        return list(logits)


def make(pages=64, page=4, max_seqs=8, budget=64, watermark=0.0, max_model_len=10_000, eos=()):
    cache = CacheManager([NEED], page_size=page, num_pages=pages, max_requests=max_seqs)
    runner = FakeRunner(cache)
    pol = StaticPolicy(max_num_seqs=max_seqs, max_batched_tokens=budget, watermark=watermark)
    eng = Engine(runner, cache, FakeSampler(), pol, max_model_len=max_model_len, eos_ids=eos)
    return eng, runner, cache


def prompt(i, n):
    return [(i * 13 + j * 7) % VOCAB for j in range(n)]


def test_first_come_first_served_and_budget_cuts_prompts():
    eng, runner, cache = make(budget=10)
    a = eng.new_sequence(prompt(0, 25), 3, ignore_eos=True)
    b = eng.new_sequence(prompt(1, 4), 3, ignore_eos=True)
    eng.step()
    assert runner.log[0] == [(a.seq_id, 10, [])]                     # first portion, no logits wanted
    eng.step()
    assert runner.log[1] == [(a.seq_id, 10, [])]
    eng.step()                                                       # a's last 5 tokens, then b is admitted
    assert runner.log[2] == [(a.seq_id, 5, [4]), (b.seq_id, 4, [3])]
    eng.step()                                                       # both decode
    assert runner.log[3] == [(a.seq_id, 1, [0]), (b.seq_id, 1, [0])]
    eng.run_until_done()
    assert a.tokens[25:] == expected(prompt(0, 25), 3) and b.tokens[4:] == expected(prompt(1, 4), 3)
    assert a.finish_reason == b.finish_reason == "length"
    cache.check()
    assert cache.num_free == cache.num_pages and not cache.stored
    c = eng.counters
    assert c["prompt_tokens_total"] == 29 and c["generation_tokens_total"] == 6 and c["request_success_total"] == 2


def test_decodes_go_first_and_prefill_takes_what_is_left():
    eng, runner, _ = make(budget=8)
    a = eng.new_sequence(prompt(0, 3), 10, ignore_eos=True)
    eng.step()
    b = eng.new_sequence(prompt(1, 20), 2, ignore_eos=True)
    eng.step()
    assert runner.log[1] == [(b.seq_id, 7, []), (a.seq_id, 1, [0])]  # 1 decode + 7 of the budget of 8 (portions are listed first)
    eng.step()
    assert runner.log[2] == [(b.seq_id, 7, []), (a.seq_id, 1, [0])]
    eng.step()
    assert runner.log[3] == [(b.seq_id, 6, [5]), (a.seq_id, 1, [0])]


def test_max_num_seqs_caps_the_running_set():
    eng, runner, _ = make(max_seqs=2, budget=100)
    seqs = [eng.new_sequence(prompt(i, 5), 4, ignore_eos=True) for i in range(5)]
    eng.step()
    assert len(runner.log[0]) == 2 and len(eng.scheduler.waiting) == 3
    eng.run_until_done()
    for i, s in enumerate(seqs):
        assert s.tokens[5:] == expected(prompt(i, 5), 4)


def test_watermark_and_head_of_line_blocking():
    eng, runner, cache = make(pages=10, page=4, budget=100, watermark=0.2)          # reserve 2 pages
    a = eng.new_sequence(prompt(0, 20), 30, ignore_eos=True)                        # 5 pages
    big = eng.new_sequence(prompt(1, 16), 2, ignore_eos=True)                       # 4 pages: 4 > 5 - 2
    small = eng.new_sequence(prompt(2, 3), 2, ignore_eos=True)                      # would fit, but waits behind `big`
    eng.step()
    assert [r for r, _, _ in runner.log[0]] == [a.seq_id]
    assert list(eng.scheduler.waiting) == [big, small]
    eng.run_until_done()
    assert big.tokens[16:] == expected(prompt(1, 16), 2) and small.tokens[3:] == expected(prompt(2, 3), 2)


def test_pages_run_out_newest_is_preempted_and_recomputed():
    eng, runner, cache = make(pages=8, page=4, budget=100)
    a = eng.new_sequence(prompt(0, 10), 14, ignore_eos=True)     # grows to 24 tokens = 6 pages
    b = eng.new_sequence(prompt(1, 10), 14, ignore_eos=True)
    eng.run_until_done()
    assert eng.counters["num_preemptions_total"] >= 1 and b.num_preemptions >= 1 and a.num_preemptions == 0
    assert a.tokens[10:] == expected(prompt(0, 10), 14) and b.tokens[10:] == expected(prompt(1, 10), 14)
    # the recomputation fed prompt + generated tokens again from position 0
    refeeds = [n for step in runner.log for r, n, _ in step if r == b.seq_id and n > 10]
    assert refeeds, "the preempted request was re-prefilled with its generated tokens"
    cache.check()
    assert cache.num_free == 8


def test_generation_does_not_depend_on_budget_pages_or_batch_cap():
    prompts = [prompt(i, n) for i, n in enumerate([1, 9, 40, 64, 130, 7, 33])]
    want = [expected(p, 12) for p in prompts]
    for pages, budget, max_seqs in [(400, 2048, 8), (60, 16, 8), (48, 7, 3), (45, 33, 8), (200, 1, 2)]:
        eng, _, cache = make(pages=pages, page=4, budget=budget, max_seqs=max_seqs, watermark=0.01)
        seqs = [eng.new_sequence(p, 12, ignore_eos=True) for p in prompts]
        eng.run_until_done()
        assert [s.tokens[s.prompt_len:] for s in seqs] == want, (pages, budget, max_seqs)
        cache.check()
        assert cache.num_free == pages


def test_lone_request_that_cannot_grow_ends_with_out_of_pages():
    eng, _, cache = make(pages=4, page=4, budget=100)
    eng.max_model_len = 1000                        # pretend the cap to the pool's size was not applied
    s = eng.new_sequence(prompt(0, 14), 50, ignore_eos=True)
    done = []
    s.on_output = lambda seq, new, fin: done.append(fin)
    eng.run_until_done()
    assert s.finished and s.finish_reason == "out_of_pages" and done[-1] is True
    assert s.tokens[14:] == expected(prompt(0, 14), 50)[:len(s.tokens) - 14]
    assert eng.counters["request_failure_total"] == 1
    cache.check()
    assert cache.num_free == 4


def test_stuck_prefills_make_room_instead_of_spinning():
    """Two half-prefilled prompts hold every page and neither can take its next portion.  The
    policy's own order of admission does not lead here (the oldest prompt takes the whole
    budget first), so the state is set up by hand; the scheduler must preempt, not spin."""
    eng, runner, cache = make(pages=10, page=4, budget=12)
    a = Sequence(seq_id=100, tokens=prompt(0, 28), max_tokens=2, ignore_eos=True)
    b = Sequence(seq_id=101, tokens=prompt(1, 28), max_tokens=2, ignore_eos=True)
    for s in (a, b):
        cache.admit(s.seq_id)
        cache.ensure(s.seq_id, 20)
        runner.history[s.seq_id] = list(s.tokens[:20])
        cache.advance(s.seq_id, 20)
        s.num_computed = 20
        eng.scheduler.running.append(s)
    assert cache.num_free == 0
    eng.run_until_done(max_steps=200)
    assert a.finished and b.finished
    assert a.tokens[28:] == expected(prompt(0, 28), 2) and b.tokens[28:] == expected(prompt(1, 28), 2)
    assert eng.counters["num_preemptions_total"] >= 1 and b.num_preemptions >= 1
    cache.check()
    assert cache.num_free == 10


def test_stop_rules():
    p = prompt(3, 6)
    full = expected(p, 40)
    eos = full[5]
    cut = full.index(eos) + 1
    eng, _, _ = make(eos=(eos,))
    s1 = eng.new_sequence(p, 40)
    s2 = eng.new_sequence(p, 40, ignore_eos=True)
    s3 = eng.new_sequence(p, 3)
    eng.run_until_done()
    assert s1.tokens[6:] == full[:cut] and s1.finish_reason == "stop"
    assert s2.tokens[6:] == full and s2.finish_reason == "length"
    assert s3.tokens[6:] == full[:3] and s3.finish_reason == "length"
    eng, _, _ = make(max_model_len=10)
    s4 = eng.new_sequence(p, 40, ignore_eos=True)
    eng.run_until_done()
    assert len(s4.tokens) == 10 and s4.finish_reason == "length"
    with pytest.raises(ValueError):
        eng.new_sequence(prompt(0, 10), 5)          # the prompt alone reaches max_model_len


def test_max_model_len_is_capped_to_the_pool():
    eng, _, _ = make(pages=5, page=4, max_model_len=1000)
    assert eng.max_model_len == 20


def test_callbacks_report_every_token_once():
    eng, _, _ = make()
    seen = []
    s = eng.new_sequence(prompt(0, 5), 6, ignore_eos=True, on_output=lambda seq, new, fin: seen.append((list(new), fin)))
    eng.run_until_done()
    assert [t for new, _ in seen for t in new] == s.tokens[5:]
    assert [fin for _, fin in seen] == [False] * 5 + [True]


# ---- lookahead: the next step is planned and launched before the one in flight is read ---------------------
class Handle:
    def __init__(self, ids):
        self.ids = ids


class LaunchSampler(FakeSampler):
    """A sampler with the launch/fetch pair: what `launch` returns stays "on the device" until it is fetched."""

    def __init__(self):
        self.unfetched = 0

    def launch(self, logits, rows):
        assert len(logits) == len(rows)
        self.unfetched += 1
        return Handle(list(logits))

    def fetch(self, handle):
        self.unfetched -= 1
        return list(handle.ids)


class FedRunner(FakeRunner):
    """Takes tokens from the previous step's ids where an entry names their rows, as the device does."""

    def __init__(self, cache):
        super().__init__(cache)
        self.fed = 0

    def step(self, entries, prev_ids=None):
        for e in entries:
            if e.source_rows is not None:
                assert prev_ids is not None
                e.tokens = [prev_ids[r] if r >= 0 else t for t, r in zip(e.tokens, e.source_rows)]
                self.fed += 1
            assert all(t >= 0 for t in e.tokens), "a placeholder reached the step function"
        return super().step(entries)


def make_ahead(pages=64, page=4, max_seqs=8, budget=64, watermark=0.0, max_model_len=10_000, eos=()):
    cache = CacheManager([NEED], page_size=page, num_pages=pages, max_requests=max_seqs)
    runner = FedRunner(cache)
    pol = StaticPolicy(max_num_seqs=max_seqs, max_batched_tokens=budget, watermark=watermark)
    eng = Engine(runner, cache, LaunchSampler(), pol, max_model_len=max_model_len, eos_ids=eos, lookahead=True)
    return eng, runner, cache


def test_lookahead_generates_the_same_tokens_under_every_schedule():
    prompts = [prompt(i, n) for i, n in enumerate([1, 9, 40, 64, 130, 7, 33])]
    lens = [12, 1, 2, 30, 5, 12, 3]
    want = [expected(p, n) for p, n in zip(prompts, lens)]
    for pages, budget, max_seqs in [(400, 2048, 8), (60, 16, 8), (48, 7, 3), (45, 33, 8), (200, 1, 2), (400, 64, 1)]:
        eng, runner, cache = make_ahead(pages=pages, page=4, budget=budget, max_seqs=max_seqs, watermark=0.01)
        seqs = [eng.new_sequence(p, n, ignore_eos=True) for p, n in zip(prompts, lens)]
        eng.run_until_done()
        assert [s.tokens[s.prompt_len:] for s in seqs] == want, (pages, budget, max_seqs)
        assert all(s.finished and s.pending_row is None for s in seqs)
        assert runner.fed > 0, "no step was launched ahead"
        assert eng.sampler.unfetched == 0
        cache.check()
        assert cache.num_free == pages


def test_lookahead_admits_and_cuts_prompts_beside_fed_decodes():
    eng, runner, cache = make_ahead(pages=200, budget=16, max_seqs=4)
    a = eng.new_sequence(prompt(0, 5), 20, ignore_eos=True)
    eng.step()                                      # a's prompt is in flight
    b = eng.new_sequence(prompt(1, 40), 4, ignore_eos=True)
    eng.step()                                      # launched ahead: a's first decode (fed) and b's first portion
    assert runner.log[-1] == [(b.seq_id, 15, []), (a.seq_id, 1, [0])]
    assert a.num_generated == 1 and a.tokens[-1] == expected(prompt(0, 5), 1)[0] and a.pending_row is None
    eng.run_until_done()
    assert a.tokens[5:] == expected(prompt(0, 5), 20) and b.tokens[40:] == expected(prompt(1, 40), 4)
    cache.check()


def test_lookahead_frees_a_slot_only_when_the_ending_request_is_collected():
    """A request about to end by length still holds its slot while its last step is in flight: the step
    launched ahead must not admit into it."""
    eng, runner, cache = make_ahead(pages=64, budget=64, max_seqs=2)
    seqs = [eng.new_sequence(prompt(i, 6), n, ignore_eos=True) for i, n in enumerate([2, 9, 3, 3])]
    eng.run_until_done()
    for i, (s, n) in enumerate(zip(seqs, [2, 9, 3, 3])):
        assert s.tokens[6:] == expected(prompt(i, 6), n)
    cache.check()
    assert cache.num_free == 64


def test_lookahead_drops_the_token_computed_past_an_eos():
    p = prompt(3, 6)
    full = expected(p, 40)
    eos = full[5]
    cut = full.index(eos) + 1
    eng, runner, cache = make_ahead(eos=(eos,))
    s1 = eng.new_sequence(p, 40)
    s2 = eng.new_sequence(prompt(4, 9), 25, ignore_eos=True)
    eng.run_until_done()
    assert s1.tokens[6:] == full[:cut] and s1.finish_reason == "stop"
    assert s2.tokens[9:] == expected(prompt(4, 9), 25)
    assert eng.counters["generation_tokens_total"] == cut + 25
    cache.check()
    assert cache.num_free == 64


def test_more_decodes_than_the_token_budget_take_turns():
    """Seven sequences decode under a budget of three tokens a step: every one advances within three steps, and all
    finish with the tokens they would have had alone."""
    eng, runner, cache = make(pages=64, page=4, max_seqs=8, budget=3)
    prompts = [prompt(i, 2) for i in range(7)]
    seqs = [eng.new_sequence(p, 9, 0.0, True) for p in prompts]
    while any(s.num_generated == 0 for s in seqs):          # prefill: three tokens a step
        eng.step()
    for _ in range(4):
        before = [len(s.tokens) for s in seqs]
        for _ in range(3):
            eng.step()
        assert all(len(s.tokens) > b or s.finished for s, b in zip(seqs, before))
    eng.run_until_done()
    assert [s.tokens[2:] for s in seqs] == [expected(p, 9) for p in prompts]
    assert cache.num_free == 64
