"""What every part of a layer has in common.

A part is built from its spec record alone (sizes and constants as parameters), declares
the tensors it needs with `parameters(spec)`, receives them with `load(tensors)` and runs on
a `StepContext` (engine/context.py) that carries the flattened batch.  No part knows which
model it is in.

Interfaces (T = tokens of the step, w = model width):
  Norm.forward(ctx, residual[T,w] f32, delta[T,w] | None, rows=None) -> normed [T or N, w]
      adds delta into residual (float32) when given, then normalises; with `rows` it only
      reads those rows and writes residual nowhere.
  PositionEncoding.encode_and_store(ctx, qkv, cache_view, slots, heads, kv_heads)
      rotates queries and keys inside `qkv` and stores keys/values at `slots` (None = no store).
  Mixer.forward(ctx, x[T,w], call) -> delta[T,w];  Mixer.cache_need() -> CacheNeed
  FeedForward.forward(ctx, x[T,w]) -> delta[T,w]
  Block.forward(ctx, residual, delta, call) -> (residual, delta)

A delta (and the qkv handed to a position encoding) may be a `kernels.PartialSums`: a matrix product
that was split along k and whose parts are still to be added.  It is only handed to a norm or a position
encoding whose class sets `takes_partial_sums = True` (the built-in ones pass it on to kernels that add the
parts while they read); for any other part `delta_for(part, delta)` adds them first.  The parts live in
scratch that the next split product overwrites, so an arrangement uses a delta before it runs another product.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def delta_for(part, delta):
    """`delta` as `part` can take it: partial sums are added now unless the part adds them itself."""
    if delta is not None and not isinstance(delta, torch.Tensor) and not getattr(part, "takes_partial_sums", False):
        return delta.sum()
    return delta


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part owns.

    shape:  full shape after assembly.
    kind:   "matrix" (used in a matrix product: stored in the engine's dtype), "table"
            (embedding rows, same rule) or "vector" (norm gains and the like: keeps a
            float32 stored type even when the engine runs in bfloat16).
    pieces: for a tensor concatenated along dim 0 from several checkpoint tensors, the
            (piece name, rows) list in order; None for a tensor stored whole.
    """
    shape: tuple
    kind: str = "matrix"
    pieces: tuple | None = None


class Part:
    """Base of all parts: parameter declaration and loading.

    `graph_safe`: True if `forward` only launches work whose addresses and launch shapes
    depend on the step's shape alone (everything that varies is read from the step's device
    arrays).  Decode steps of a model whose parts are all graph-safe are replayed from
    captured CUDA graphs; a part that decides anything on the host per step (loops over
    requests, reads `ctx.starts`) must leave it False."""

    graph_safe = False

    @classmethod
    def parameters(cls, spec) -> dict:
        return {}

    def load(self, tensors: dict) -> None:
        for name, t in tensors.items():
            setattr(self, name, t)
