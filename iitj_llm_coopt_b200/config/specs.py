"""Architecture-neutral descriptions of what a model is made of.

A model is a list of layers and an order in which they run.  Each layer names its
parts (norm, mixer, feed-forward, position encoding) with every size and constant
they need.  Nothing here knows about a particular architecture: an architecture's
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
    """One block: `arrangement` names how the parts are wired (parts.ARRANGEMENTS)."""
    arrangement: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec


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

    def cache_entries(self) -> int:
        """Number of distinct cache entries the run order writes."""
        return len({c.cache for c in self.order if c.write})
