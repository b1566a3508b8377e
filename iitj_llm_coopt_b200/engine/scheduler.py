"""Continuous-batching scheduler.

Three phases per step, as the reference's Scheduler.schedule (engine/engine.py:91-155):
  1. decodes first: every running sequence with exactly one token left to feed; if their
     new pages do not fit, the policy's victim (the newest running sequence) is preempted
     until they do or only one sequence runs; if there are more of them than the token budget,
     they take turns from step to step;
  2. running prefills, oldest first, each cut to what is left of the step's token budget;
     a portion whose pages do not fit is skipped this step;
  3. admissions from the waiting queue while the budget, `max_num_seqs` and the page
     watermark allow; the first request that does not fit stops admission.
Token bookkeeping (engine/engine.py:8-11): `tokens` = prompt + generated, the cache holds the
first `num_computed`; decoding is "one remaining token"; a preempted sequence is recomputed
from position 0 as one (chunked) prefill of prompt + generated.

When pages run out:
  * a decode that cannot grow preempts the newest running sequence (recompute later);
  * a lone sequence that cannot grow raises OutOfPages out of `schedule`; the engine ends
    that request with finish_reason "out_of_pages" instead of stopping the process;
  * if nothing at all could be planned although sequences are running (several half
    prefilled prompts holding all pages), the newest is preempted until the rest can
    move: the reference would spin on an empty plan here;
  * the watermark is waived while nothing is running, so a prompt that fits the pool is
    always admitted eventually.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

from ..cache import OutOfPages


@dataclass
class Sequence:
    seq_id: int
    tokens: list
    max_tokens: int
    temperature: float = 0.0
    ignore_eos: bool = False
    seed: int | None = None             # request seed of its random draws (default: seq_id)
    arrival: float = field(default_factory=time.perf_counter)
    on_output: object = None            # callback(seq, new_tokens, finished)
    prompt_len: int = 0
    num_computed: int = 0               # tokens whose keys/values are in the cache
    first_token_time: float | None = None
    finish_time: float | None = None
    finished: bool = False
    finish_reason: str | None = None
    num_preemptions: int = 0
    pending_row: int | None = None      # row of the step in flight whose sampled id is this sequence's last token

    def __post_init__(self):
        self.prompt_len = self.prompt_len or len(self.tokens)

    @property
    def num_generated(self) -> int:
        return len(self.tokens) - self.prompt_len

    @property
    def remaining(self) -> int:
        return len(self.tokens) - self.num_computed


@dataclass
class Plan:
    chunks: list = field(default_factory=list)    # (seq, end): feed tokens[num_computed:end]
    decodes: list = field(default_factory=list)   # sequences with exactly one remaining token

    def __bool__(self):
        return bool(self.chunks or self.decodes)


class Scheduler:
    def __init__(self, cache, policy, counters: dict | None = None, engine=None):
        self.cache, self.policy, self.engine = cache, policy, engine
        self.counters = counters if counters is not None else {"num_preemptions_total": 0}
        self.waiting: deque = deque()
        self.running: list = []
        self.held_slots = 0          # request slots held by sequences that are not in `running` (about to finish)
        self._decode_turn = 0        # where phase 1 starts in the list of decodes when the budget cannot take them all

    def _preempt(self, seq) -> None:
        """Drop the victim's cache; it is recomputed from position 0 when re-admitted."""
        self.running.remove(seq)
        self.cache.release(seq.seq_id)
        seq.num_computed = 0
        seq.num_preemptions += 1
        self.counters["num_preemptions_total"] = self.counters.get("num_preemptions_total", 0) + 1
        self.waiting.appendleft(seq)

    def schedule(self) -> Plan:
        while True:
            plan = self._schedule_once()
            if plan or len(self.running) <= 1:
                return plan
            # sequences are running but none can move: make room
            self._preempt(self.policy.preempt_victim(self.running))

    def _schedule_once(self) -> Plan:
        cache, pol = self.cache, self.policy
        plan, budget = Plan(), pol.max_batched_tokens

        # 1. decodes: reserve one more token each, preempting the newest if pages are short
        while True:
            decodes = [s for s in self.running if s.remaining == 1]
            if cache.can_grow_all([(s.seq_id, len(s.tokens)) for s in decodes]) or len(self.running) <= 1:
                break
            self._preempt(pol.preempt_victim(self.running))
        if len(decodes) > budget:
            # more sequences decode than a step may hold tokens: start where the last step stopped, so that every
            # sequence advances within ceil(len / budget) steps (the reference always starts at the front,
            # engine/engine.py:109-112, and would starve the tail)
            at = self._decode_turn % len(decodes)
            decodes = decodes[at:] + decodes[:at]
            self._decode_turn = at + budget
        for s in decodes:
            if budget <= 0:
                break
            try:
                cache.ensure(s.seq_id, len(s.tokens))
            except OutOfPages as e:                     # only a lone sequence gets here: it cannot grow
                e.seq = s
                raise
            plan.decodes.append(s)
            budget -= 1

        # 2. running prefills, oldest first
        for s in self.running:
            if s.remaining > 1 and budget > 0:
                end = s.num_computed + min(s.remaining, budget)
                if not cache.can_fit(s.seq_id, end):
                    continue
                cache.ensure(s.seq_id, end)
                plan.chunks.append((s, end))
                budget -= end - s.num_computed

        # 3. admissions
        while self.waiting and budget > 0 and len(self.running) + self.held_slots < pol.max_num_seqs:
            i = pol.pick_next(self.waiting, self.engine)
            s = self.waiting[i]
            end = s.num_computed + min(s.remaining, budget)
            # (the watermark is waived while nothing runs, so that a prompt that fits the pool is admitted eventually)
            if not cache.can_admit(end, pol.watermark if self.running else 0.0) or not pol.admit(s, self.engine):
                break
            del self.waiting[i]
            self.running.append(s)
            cache.admit(s.seq_id)
            cache.ensure(s.seq_id, end)
            if s.remaining == 1:
                plan.decodes.append(s)
                budget -= 1
            else:
                plan.chunks.append((s, end))
                budget -= end - s.num_computed
        return plan
