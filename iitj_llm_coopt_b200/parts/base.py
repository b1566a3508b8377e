"""What every part of a layer has in common.

A part is built from its spec record alone (sizes and constants as parameters), declares
the tensors it needs with `parameters(spec)`, receives them with `load(tensors)` and runs on
a `StepContext` (engine/context.py) that carries the flattened batch.  No part knows which
model it is in.

Constructors: a norm, feed-forward, embedding or head is built as cls(spec, kernels, dtype); a position encoding
as cls(spec, kernels, dtype, device); a mixer as cls(spec, kernels, dtype, position=<its position part or None>).

Interfaces (T = tokens of the step, w = model width):
  Norm.forward(ctx, residual[T,w] f32, delta[T,w] | None, rows=None) -> normed [T or N, w]
      adds delta into residual (float32) when given, then normalises; with `rows` it only
      reads those rows and writes residual nowhere.
  PositionEncoding.encode_and_store(ctx, qkv, cache_view, slots, heads, kv_heads)
      rotates queries and keys inside `qkv` and stores keys/values at `slots` (None = no store).
  Mixer.forward(ctx, x[T,w], call) -> delta[T,w];  Mixer.cache_need() -> CacheNeed
  FeedForward.forward(ctx, x[T,w]) -> delta[T,w]
  Embedding.forward(ctx) -> residual[T,w] f32;   Head.forward(ctx, x[N,w]) -> logits[N,vocab] f32
  Arrangement.forward(ctx, residual, delta, call) -> (residual, delta)     (parts/block.py)

Per-step index arrays of a part's own.  The step function builds the arrays every part needs (positions, block
tables, cache slots, ...: engine/context.py) and copies them to the device in one buffer.  A part whose kernels
need more than those (tile lists, per-request work items) implements `prepare_step(shape) -> StepPlan | None`:
it is called on the host once per step (once for all parts that share a `prepare_key`), before the copy, with
the step's `StepShape`; the int32 arrays it returns travel in the same buffer, come back to it as device views
through `StepPlan.bind`, and its forward finds the plan in `ctx.prepared[prepare_key]`.  Whatever of the plan a
captured CUDA graph freezes (a launch shape, a split count) goes into `StepPlan.graph_key`, so a step with another
value is captured anew.

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


@dataclass
class StepShape:
    """What a part's `prepare_step` is told about the step (host side, before anything is copied)."""
    query_lens: list             # tokens each request brings
    seq_lens: list               # tokens each request holds after the step
    num_tokens: int
    decode_shaped: bool          # every request brings one token and wants its logits
    graphable: bool              # the step may be captured into, or replayed from, a CUDA graph
    device: object


class StepPlan:
    """A part's own per-step index arrays: `arrays` {name: int32 numpy array or list} go into the step's one
    staging buffer; `graph_key` is what a captured graph of this step freezes; `bind(views)` receives the arrays
    as device tensors (same names) after the copy was issued."""

    def __init__(self, arrays: dict | None = None, graph_key=()):
        self.arrays, self.graph_key = arrays or {}, graph_key
        self.device_arrays: dict = {}

    def bind(self, views: dict) -> None:
        self.device_arrays = views


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
    part_name = ""           # the part's name in its arrangement (set by the model builder)
    prepare_key = None       # parts with the same key share one `prepare_step` call (and one StepPlan) per step

    @classmethod
    def parameters(cls, spec) -> dict:
        return {}

    def subparts(self) -> tuple:
        """Parts this part owns (a mixer's position encoding): they count toward `graph_safe` and are asked for
        their `prepare_step` too."""
        return ()

    def prepare_step(self, shape):
        """Per-step index arrays of this part's own (see the module text); None if it needs none."""
        return None

    def load(self, tensors: dict) -> None:
        for name, t in tensors.items():
            setattr(self, name, t)
