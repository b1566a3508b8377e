"""The engine: scheduler above the step function, sampling, stop rules, counters.

One `step()` is the reference's Engine.step (engine/engine.py:407-515) without its draft
phase: plan, turn the plan into step entries (a prefill portion feeds
tokens[num_computed:end]; a decode feeds the last token), run the step function, sample
where a request reached the end of its tokens, append with the stop rules
(engine/engine.py:293-308: max_tokens -> "length", EOS unless ignore_eos -> "stop",
max_model_len -> "length"), finish and free.  Logits are asked for only at rows that are
sampled: a prompt portion that does not reach the prompt's end wants none.
"""
from __future__ import annotations

import time

import torch

from ..cache import OutOfPages
from .policy import StaticPolicy
from .runner import StepEntry
from .scheduler import Plan, Scheduler, Sequence

PLACEHOLDER = -1       # stands in a token list for the token that the step in flight is sampling

COUNTERS = ("prompt_tokens_total", "generation_tokens_total", "num_preemptions_total",
            "request_success_total", "request_failure_total", "steps_total", "step_seconds_total")


class Engine:
    def __init__(self, runner, cache, sampler, policy=None, max_model_len: int = 32768, eos_ids=(),
                 lookahead: bool = False):
        self.runner, self.cache, self.sampler = runner, cache, sampler
        self.lookahead = bool(lookahead) and hasattr(sampler, "launch")
        self._inflight = None
        self.policy = policy or StaticPolicy()
        self.eos_ids = set(eos_ids)
        self.max_model_len = max_model_len
        self.kv_capacity_tokens = cache.capacity_tokens
        if self.kv_capacity_tokens < self.max_model_len:
            # as engine/engine.py:216-219: a lone sequence must always fit the pool
            self.max_model_len = self.kv_capacity_tokens
        if self.policy.max_num_seqs > cache.max_requests:
            raise ValueError(f"max_num_seqs {self.policy.max_num_seqs} exceeds the cache's "
                             f"{cache.max_requests} request slots")
        self.counters = {k: 0 for k in COUNTERS}
        self.gauges: dict = {}
        self.scheduler = Scheduler(cache, self.policy, self.counters, engine=self)
        self._next_id = 0

    # ---- request lifecycle ---------------------------------------------------------------
    def add_request(self, seq: Sequence) -> Sequence:
        if not seq.tokens:
            raise ValueError("a request needs at least one prompt token")
        if len(seq.tokens) >= self.max_model_len:
            raise ValueError(f"prompt of {len(seq.tokens)} tokens does not fit max_model_len {self.max_model_len}")
        self.scheduler.waiting.append(seq)
        return seq

    def new_sequence(self, prompt, max_tokens, temperature=0.0, ignore_eos=False, seed=None, on_output=None):
        seq = Sequence(seq_id=self._next_id, tokens=list(prompt), max_tokens=max_tokens, temperature=temperature,
                       ignore_eos=ignore_eos, seed=seed, on_output=on_output)
        self._next_id += 1
        return self.add_request(seq)

    def release(self, seq) -> None:
        if self.cache.has(seq.seq_id):
            self.cache.release(seq.seq_id)

    def _finish(self, seq, reason) -> None:
        seq.finished, seq.finish_reason = True, reason
        seq.finish_time = time.perf_counter()
        if seq in self.scheduler.running:
            self.scheduler.running.remove(seq)
        self.release(seq)
        key = "request_failure_total" if reason == "out_of_pages" else "request_success_total"
        self.counters[key] += 1

    def _append(self, seq, new_tokens) -> list:
        """Append sampled tokens under the stop rules; returns those kept."""
        kept = []
        for t in new_tokens:
            seq.tokens.append(t)
            kept.append(t)
            if seq.num_generated >= seq.max_tokens:
                seq.finish_reason = "length"
                break
            if not seq.ignore_eos and t in self.eos_ids:
                seq.finish_reason = "stop"
                break
            if len(seq.tokens) >= self.max_model_len:
                seq.finish_reason = "length"
                break
        return kept

    # ---- one step ------------------------------------------------------------------------
    # A step is launched (scheduler, step function, sampling kernel, copy of the ids to the host) and
    # collected (ids read, tokens appended, stop rules, finish and free).  Without lookahead `step()` does
    # both.  With lookahead a launched step stays in flight, and the next `step()` first plans and launches
    # its successor and only then collects the step in flight, so the GPU never waits for the host.  The
    # successor is planned as if the step in flight had already handed every sequence its token: a
    # placeholder stands in the token list, and the successor takes that token from the sampled ids on the
    # device.  Stops by max_tokens and max_model_len are known beforehand (those sequences are left out); a
    # stop by EOS is seen one step late, and the token the successor computed for that sequence is dropped.
    # The successor is only launched when its decodes need no preemption; else the step in flight is
    # collected first and the scheduler decides with everything known.
    def step(self) -> bool:
        prev = self._inflight
        if prev is not None:
            nxt = self._launch_ahead(prev) if self.lookahead and hasattr(prev["handle"], "ids") else None
            self._inflight = None
            self._collect(prev)
            self._inflight = nxt
            return True
        try:
            plan = self.scheduler.schedule()
        except OutOfPages as e:
            seq = getattr(e, "seq", None)
            if seq is None:
                raise
            self._finish(seq, "out_of_pages")
            if seq.on_output:
                seq.on_output(seq, [], True)
            return True
        if not plan:
            return False
        rec = self._launch(plan)
        if self.lookahead:
            self._inflight = rec
        else:
            self._collect(rec)
        return True

    def _launch(self, plan, prev_ids=None) -> dict:
        t0 = time.perf_counter()
        entries, sampled = [], []         # sampled: sequences whose last fed token wants logits
        for s, end in plan.chunks:
            toks = s.tokens[s.num_computed:end]
            last = end == len(s.tokens)
            entries.append(StepEntry(s.seq_id, toks, [len(toks) - 1] if last else []))
            if last:
                sampled.append(s)
        for s in plan.decodes:
            if s.tokens[-1] == PLACEHOLDER:       # the step in flight is about to sample it: fed on the device
                entries.append(StepEntry(s.seq_id, [0], [0], source_rows=[s.pending_row]))
            else:
                entries.append(StepEntry(s.seq_id, [s.tokens[-1]], [0]))
            sampled.append(s)
        logits = self.runner.step(entries, prev_ids=prev_ids) if prev_ids is not None else self.runner.step(entries)
        for s, end in plan.chunks:
            self.counters["prompt_tokens_total"] += end - s.num_computed
            s.num_computed = end
        return self._sample(logits, sampled, [s.num_generated for s in sampled], sum(len(e.tokens) for e in entries), t0)

    def _sample(self, logits, sampled, token_index, n_tokens, t0) -> dict:
        handle = None
        if sampled:
            rows = [(s.temperature, s.seq_id if s.seed is None else s.seed, i) for s, i in zip(sampled, token_index)]
            if hasattr(self.sampler, "launch"):
                handle = self.sampler.launch(logits, rows)
            else:
                handle = list(self.sampler.sample(logits, rows))
        return {"sampled": sampled, "handle": handle, "n_tokens": n_tokens, "t0": t0}

    def _ends_by_length(self, s, extra: int = 1) -> bool:
        """True if the sequence stops for length once `extra` more tokens are appended."""
        return s.num_generated + extra >= s.max_tokens or len(s.tokens) + extra >= self.max_model_len

    def _launch_ahead(self, prev):
        """Plans and launches the step after `prev` while `prev` is still in flight; None if that cannot be done
        without knowing prev's tokens (then nothing has changed)."""
        sched, cache = self.scheduler, self.cache
        cont = [(i, s) for i, s in enumerate(prev["sampled"]) if not s.finished and not self._ends_by_length(s)]
        ending = [s for s in prev["sampled"] if not s.finished and self._ends_by_length(s)]
        running_before = list(sched.running)
        saved = [(s, s.num_computed) for _, s in cont]
        for i, s in cont:                          # as if prev had handed over its tokens
            s.tokens.append(PLACEHOLDER)
            s.num_computed = len(s.tokens) - 1
            s.pending_row = i
        for s in ending:                           # they finish when prev is collected: not to be planned
            if s in sched.running:
                sched.running.remove(s)

        def undo():
            for s, n in saved:
                s.tokens.pop()
                s.num_computed, s.pending_row = n, None
            sched.running[:] = running_before
            return None

        decodes = [s for s in sched.running if s.remaining == 1]
        if not cache.can_grow_all([(s.seq_id, len(s.tokens)) for s in decodes]):
            return undo()                          # somebody would have to give way: decide that with prev known
        waiting_before = len(sched.waiting)
        sched.held_slots = len(running_before) - len(sched.running)     # the ending ones keep slot and pages until collected
        try:
            plan = sched._schedule_once()
        finally:
            sched.held_slots = 0
        if not plan:
            if len(sched.waiting) != waiting_before:
                raise RuntimeError("the scheduler admitted a request without planning it")
            return undo()
        return self._launch(plan, prev_ids=prev["handle"].ids)

    def _collect(self, rec) -> None:
        sampled, handle = rec["sampled"], rec["handle"]
        new_tokens = []
        if sampled:
            new_tokens = self.sampler.fetch(handle) if hasattr(self.sampler, "fetch") else handle
        now = time.perf_counter()
        for s, tok in zip(sampled, new_tokens):
            if s.finished:
                continue                  # it ended at EOS one step ago; this token was computed in vain
            if s.pending_row is not None:
                # the step after this one is already in flight and counts on this token: it takes the
                # placeholder's place; length stops were ruled out before, EOS is what can still end it
                s.tokens[-1], s.pending_row = tok, None
                kept = [tok]
                if not s.ignore_eos and tok in self.eos_ids:
                    s.finish_reason = "stop"
            else:
                kept = self._append(s, [tok])
                s.num_computed = len(s.tokens) - 1      # everything but the newly sampled token is cached
            self.counters["generation_tokens_total"] += len(kept)
            if s.first_token_time is None:
                s.first_token_time = now
            done = s.finish_reason is not None
            if done:
                self._finish(s, s.finish_reason)
            if s.on_output:
                s.on_output(s, kept, done)
        end_t = time.perf_counter()
        self.counters["steps_total"] += 1
        self.counters["step_seconds_total"] += end_t - rec["t0"]
        self.gauges = {
            "num_requests_running": len(self.scheduler.running),
            "num_requests_waiting": len(self.scheduler.waiting),
            "kv_cache_usage_perc": self.cache.usage,
            "kv_capacity_tokens": self.kv_capacity_tokens,
            "step_time_s": end_t - rec["t0"],
            "batch_tokens": rec["n_tokens"],
            **self.policy.state(),
        }

    def has_work(self) -> bool:
        return bool(self.scheduler.running or self.scheduler.waiting or self._inflight is not None)

    def run_until_done(self, max_steps: int | None = None) -> int:
        """The reference's worker loop (engine/worker.py:64-65) in-process."""
        steps = 0
        while self.has_work():
            if not self.step():
                raise RuntimeError("scheduler made no progress although requests are pending")
            steps += 1
            if max_steps is not None and steps >= max_steps:
                break
        return steps
