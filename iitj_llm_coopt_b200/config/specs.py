"""Architecture-neutral descriptions of what a model is made of.

A model is an embedding, a list of layers, an order in which they run, a final norm and an
output head.  Each layer names its arrangement and, by name, the parts that arrangement is wired
from (norms, a mixer, a feed-forward, ...; a mixer names its position encoding) with every size
and constant they need.  Nothing here knows about a particular architecture: an architecture's
typed configuration (for instance `LlamaConfig`) turns its config.json keys into
these records, and the parts are built from the records alone.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class NormSpec:
    kind: str                    # key in parts.NORMS
    width: int
    eps: float
    options: tuple = ()          # extra (name, value) pairs for other norm kinds


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer."""
    kind: str                    # key in parts.POSITION_ENCODINGS ("rope", "none", ...)
    head_dim: int
    rotary_dim: int              # leading dims of each head that are rotated
    theta: float = 10000.0
    scaling: tuple = ()          # sorted (name, value) pairs of the scaling law, () if none
    max_position: int = 0

    def scaling_dict(self) -> dict:
        return dict(self.scaling)


@dataclass(frozen=True)
class CacheNeed:
    """What one layer keeps per request between steps.

    kind "paged_kv": `kv_heads * head_dim` keys and as many values per token, in pages.
        window == 0 keeps every token, window > 0 only the last `window` tokens.
    kind "state":    a fixed-size record per request (`state_shape`, `state_dtype`).
    kind "none":     nothing.
    Layers whose needs compare equal share one group of the cache manager.
    """
    kind: str = "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: tuple = ()
    state_dtype: str = "float32"


@dataclass(frozen=True)
class MixerSpec:
    kind: str                    # key in parts.MIXERS
    width: int
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0              # 0 = all earlier tokens
    softmax_scale: float = 0.0   # 0 = 1/sqrt(head_dim)
    position: PositionSpec | None = None
    options: tuple = ()

    def option(self, name: str, default: Any = None) -> Any:
        return dict(self.options).get(name, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                    # key in parts.FEED_FORWARDS
    width: int
    inner: int
    activation: str = "silu"
    experts: int = 0             # 0 = dense
    experts_per_token: int = 0
    options: tuple = ()

    def option(self, name: str, default: Any = None) -> Any:
        return dict(self.options).get(name, default)


@dataclass(frozen=True)
class LayerSpec:
    """One block: `arrangement` names how the parts are wired (parts.ARRANGEMENTS); `parts` holds one spec record
    for each part name the arrangement declares (its PARTS), as (name, spec) pairs.  `LayerSpec.of("prenorm",
    mixer_norm=..., mixer=..., feed_forward_norm=..., feed_forward=...)` builds one from keywords."""
    arrangement: str
    parts: tuple = ()            # of (part name, spec record)

    @classmethod
    def of(cls, arrangement: str, **parts) -> "LayerSpec":
        return cls(arrangement, tuple(parts.items()))

    def part(self, name: str):
        for n, spec in self.parts:
            if n == name:
                return spec
        raise KeyError(f"layer ({self.arrangement}) has no part {name!r}; it has: {', '.join(n for n, _ in self.parts)}")

    def names(self) -> tuple:
        return tuple(n for n, _ in self.parts)


@dataclass(frozen=True)
class EmbeddingSpec:
    """How token ids become the first residual stream."""
    kind: str                    # key in parts.EMBEDDINGS
    vocab: int
    width: int
    scale: float = 1.0
    options: tuple = ()


@dataclass(frozen=True)
class HeadSpec:
    """How the normed rows that want logits become logits."""
    kind: str                    # key in parts.HEADS
    vocab: int
    width: int
    scale: float = 1.0
    options: tuple = ()


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    layer:  index into ModelSpec.layers (a layer may be named more than once).
    cache:  index of the cache entry the mixer reads; normally the call's own index
            in the run order, another call's index to read that call's cache.
    write:  whether this call stores its new keys/values/state in that entry.
    """
    layer: int
    cache: int
    write: bool = True


@dataclass(frozen=True)
class ModelSpec:
    width: int
    vocab: int
    layers: tuple                # of LayerSpec
    order: tuple                 # of LayerCall
    final_norm: NormSpec
    tie_embeddings: bool
    max_position: int
    eos_token_ids: tuple = ()
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    embedding: EmbeddingSpec | None = None     # None: a plain table of [vocab, width] scaled by embedding_scale
    head: HeadSpec | None = None               # None: a plain [vocab, width] projection scaled by logit_scale

    def embedding_spec(self) -> EmbeddingSpec:
        return self.embedding or EmbeddingSpec("table", self.vocab, self.width, self.embedding_scale)

    def head_spec(self) -> HeadSpec:
        return self.head or HeadSpec("linear", self.vocab, self.width, self.logit_scale)

    def cache_entries(self) -> int:
        """Number of distinct cache entries the run order writes."""
        return len({c.cache for c in self.order if c.write})
