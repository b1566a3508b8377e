"""Per-request sampling options.

The reference's per-request knobs are `max_tokens`, `temperature` (0 = greedy) and
`ignore_eos` (engine/engine.py:33-41); it has no top-k, top-p or penalties
(engine/spec_decode.py:12-17).  `seed` is added so that a request's random draws can be
fixed independently of the engine's seed and of what else is running.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0
    ignore_eos: bool = False
    seed: int | None = None

    def __post_init__(self):
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
