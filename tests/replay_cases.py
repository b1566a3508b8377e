"""Generators of replay traces: the same requests cut in different ways.

A trace is a list of steps; a step is (entries, ends) with entries = [(request id, tokens,
wanted places)] and ends = request ids that finish after the step.  Every position of
every request is wanted somewhere, so each way of cutting yields the full set of logits.
"""
import random


def requests_for(vocab, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def whole(reqs):
    """Each request alone and whole."""
    return [([(rid, toks, list(range(len(toks))))], [rid]) for rid, toks in reqs.items()]


def last_one_by_one(reqs, tail=32):
    """Most of a request in one step, then its last `tail` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        head = max(len(toks) - tail, 0)
        if head:
            steps.append(([(rid, toks[:head], list(range(head)))], []))
        for i in range(head, len(toks)):
            steps.append(([(rid, toks[i:i + 1], [0])], [rid] if i == len(toks) - 1 else []))
    return steps


PORTIONS = [7, 2, 13, 2, 5, 3, 16, 2, 31, 2, 17, 4, 64, 2, 9]


def portions(reqs, sizes=PORTIONS):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in reqs.items():
        i, j = 0, 0
        while i < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - i)
            j += 1
            steps.append(([(rid, toks[i:i + n], list(range(n)))], [rid] if i + n == len(toks) else []))
            i += n
    return steps


def mixed(reqs, live=4, decode_tail=9, seed=0, sizes=PORTIONS):
    """Up to `live` requests at a time: portions of some beside single tokens of others in one
    step, requests now and then left out of a step; a finished request's place goes to the
    next one.  Returns (steps, the largest sum over live requests of tokens rounded up to 64)."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    active = {}                      # rid -> [tokens, consumed, index into sizes]
    steps, peak = [], 0
    while waiting or active:
        while waiting and len(active) < live:
            rid, toks = waiting.pop(0)
            active[rid] = [toks, 0, rng.randrange(len(sizes))]
        peak = max(peak, sum(-(-len(v[0]) // 64) * 64 for v in active.values()))
        entries, ends = [], []
        for rid, rec in list(active.items()):
            toks, done, j = rec
            if len(active) > 1 and rng.random() < 0.2:
                continue             # left out of this step
            head = max(len(toks) - decode_tail, 0)
            if done < head:
                n = min(sizes[j % len(sizes)], head - done)
                rec[2] += 1
            else:
                n = 1
            entries.append((rid, toks[done:done + n], list(range(n))))
            rec[1] = done + n
            if rec[1] == len(toks):
                ends.append(rid)
                del active[rid]
        if entries:
            steps.append((entries, ends))
    return steps, peak


def as_jsonl(steps):
    """The trace as the lines bin/trace_run reads."""
    import json
    return [json.dumps({"step": i, "entries": [{"id": rid, "tokens": toks, "want": want} for rid, toks, want in entries],
                        "end": ends}) for i, (entries, ends) in enumerate(steps)]
