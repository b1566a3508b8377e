"""The static policy: the only place the scheduler's knobs and choices live.

Same knobs and hooks as the reference's StaticPolicy (engine/policy.py:10-52):
`max_num_seqs` 256, `max_batched_tokens` (8192 there; its server passes 2048,
engine/server.py:189-190), `watermark` 0.01, first-come-first-served `pick_next`, the newest
running sequence as `preempt_victim`, `admit` always true.  The speculative-decoding and
tiering knobs of the reference are not carried.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class StaticPolicy:
    max_num_seqs: int = 256
    max_batched_tokens: int = 2048
    watermark: float = 0.01

    name = "static"

    def admit(self, seq, engine) -> bool:
        return True

    def pick_next(self, waiting, engine) -> int:
        """Index of the waiting request to admit next (first come, first served)."""
        return 0

    def preempt_victim(self, running: list):
        """The newest running sequence gives way."""
        return running[-1]

    def state(self) -> dict:
        return {"max_num_seqs": self.max_num_seqs, "max_batched_tokens": self.max_batched_tokens}
