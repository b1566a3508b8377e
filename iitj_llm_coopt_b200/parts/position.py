"""Position encodings applied to queries and keys inside a mixer.

`RotaryEmbedding`: half-split rotation (engine/model.py:92-94, 199-200) with inverse
frequencies 1 / theta^(2i/d) and the optional llama3 scaling law (engine/model.py:68-82).
The frequencies are computed once in float32 on the host with the reference's formula; the
angle position * inv_freq and its sine and cosine are evaluated in float32 inside the
kernel for every token, so no table of max_position rows exists and none is rounded to
the model's type.

`NoPosition` leaves queries and keys as they are and only stores keys and values.
"""
from __future__ import annotations

import math

import torch

from .base import Part


def rope_inverse_frequencies(rotary_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """float32 [rotary_dim/2]; llama3 scaling as engine/model.py:71-82."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.int64).float() / rotary_dim))
    if not scaling or scaling.get("rope_type", scaling.get("type")) != "llama3":
        return inv_freq
    factor, lo, hi = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    old = scaling["original_max_position_embeddings"]
    low_wavelen, high_wavelen = old / lo, old / hi
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old / wavelen - lo) / (hi - lo)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, scaled).float()


class RotaryEmbedding(Part):
    graph_safe = True
    takes_partial_sums = True     # encode_and_store adds the k-split parts of the qkv product as it reads them

    def __init__(self, spec, kernels, dtype, device="cuda"):
        self.spec, self.k = spec, kernels
        self.head_dim, self.rotary_dim = spec.head_dim, spec.rotary_dim
        self.inv_freq = rope_inverse_frequencies(spec.rotary_dim, spec.theta, spec.scaling_dict()).to(device)

    def tables(self, ctx):
        """cos and sin of this step's positions, computed by the first layer that asks and shared by
        every layer with the same position spec."""
        key = ("rope", self.spec)
        tabs = ctx.shared.get(key)
        if tabs is None:
            half = self.rotary_dim // 2
            name = f"rope.{hash(self.spec) & 0xffffffff:x}"
            cos = ctx.buffer(name + ".cos", (ctx.num_tokens, half), torch.float32)
            sin = ctx.buffer(name + ".sin", (ctx.num_tokens, half), torch.float32)
            tabs = ctx.shared[key] = self.k.rope_tables(ctx.positions, self.inv_freq, cos, sin)
        return tabs

    def encode_and_store(self, ctx, qkv, cache_view, slots, heads, kv_heads):
        return self.k.rope_store(qkv, ctx.positions, self.inv_freq, slots, cache_view, heads, kv_heads,
                                 self.head_dim, self.rotary_dim, tables=self.tables(ctx) if self.rotary_dim else None)

    def decode_tables(self, ctx):
        """(cos, sin) for a mixer whose decode kernel rotates and stores by itself, or None if this encoding
        cannot be handed over like that (only part of the head is rotated)."""
        return self.tables(ctx) if self.rotary_dim == self.head_dim else None


class NoPosition(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype, device="cuda"):
        self.spec, self.k, self.head_dim = spec, kernels, spec.head_dim

    def encode_and_store(self, ctx, qkv, cache_view, slots, heads, kv_heads):
        if slots is not None:
            self.k.rope_store(qkv, ctx.positions, None, slots, cache_view, heads, kv_heads, self.head_dim, 0)
