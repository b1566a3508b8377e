"""Token mixers.

`PagedAttention`: grouped-query causal attention over a paged key/value cache.
    qkv = x Wqkv^T (no bias; Wqkv = [Wq; Wk; Wv], engine/model.py:113-114, 194-198), position
    encoding on q and k, keys/values of the new tokens stored in the cache
    (engine/model.py:201-203), softmax(scale * q k^T) over the request's visible keys with
    scale = 1/sqrt(head_dim) unless the spec gives one (engine/model.py:102, 204-207),
    out = (P v) Wo^T (engine/model.py:208).
The mixer reads whichever cache entry the run order hands it (`call.cache`) and stores its
own keys and values there only if `call.write` is set, so a layer can read another
layer's cache.
"""
from __future__ import annotations

from ..config.specs import CacheNeed
from ..kernels import materialize
from .base import ParamSpec, Part


class PagedAttention(Part):
    graph_safe = True
    prepare_key = "paged_attention"      # every attention layer of a model shares one plan of the step's tiles and items

    def __init__(self, spec, kernels, dtype, position):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.heads, self.kv_heads, self.head_dim = spec.width, spec.heads, spec.kv_heads, spec.head_dim
        if self.heads % self.kv_heads:
            raise ValueError(f"attention: heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.window, self.scale = spec.window, spec.softmax_scale
        self.position = position
        self.qkv_width = (self.heads + 2 * self.kv_heads) * self.head_dim
        self.qkv = self.o = None

    @classmethod
    def parameters(cls, spec) -> dict:
        q, kv = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
        return {
            "qkv": ParamSpec((q + 2 * kv, spec.width), pieces=(("q", q), ("k", kv), ("v", kv))),
            "o": ParamSpec((spec.width, q)),
        }

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="paged_kv", kv_heads=spec.kv_heads, head_dim=spec.head_dim, window=spec.window)

    def subparts(self) -> tuple:
        return (self.position,) if self.position is not None else ()

    def prepare_step(self, shape):
        """The kernel set's plan of this step's attention work (which tokens are single decoded tokens, how prompt
        portions are cut into query tiles, what a captured graph freezes of it); None for a kernel set that plans
        nothing on the host."""
        plan = getattr(self.k, "plan_attention", None)
        return plan(shape) if plan is not None else None

    def forward(self, ctx, x, call):
        t = x.shape[0]
        group, view = ctx.cache.view(call.cache)
        meta = ctx.group(group)
        plan = ctx.prepared.get(self.prepare_key)
        if plan is not None:
            meta.attention_plan = plan
        qkv = ctx.buffer("attn.qkv", (t, self.qkv_width), self.dtype)
        # a position encoding that says so takes the product's k-split partial sums and adds them as it reads
        qkv = self.k.linear(x, self.qkv, qkv, defer=getattr(self.position, "takes_partial_sums", False))
        attn = ctx.buffer("attn.ctx", (t, self.heads * self.head_dim), self.dtype)
        # A step of single decoded tokens whose position encoding hands over its tables: the attention kernel adds
        # the product's parts, rotates, stores key and value, and attends (one kernel boundary less per layer).
        tables = None
        fused = getattr(self.k, "can_fuse_decode", None)
        if call.write and fused is not None and hasattr(self.position, "decode_tables") and \
                fused(qkv, meta, view, self.heads, self.kv_heads, self.head_dim):
            tables = self.position.decode_tables(ctx)
        if tables is not None:
            self.k.attention_decode_fused(qkv, tables, meta.slots, view, meta, attn, self.heads, self.kv_heads,
                                          self.head_dim, window=self.window, scale=self.scale)
        else:
            rotated = self.position.encode_and_store(ctx, qkv, view, meta.slots if call.write else None,
                                                     self.heads, self.kv_heads)
            qkv = rotated if rotated is not None else materialize(qkv)
            self.k.attention(qkv, view, meta, attn, self.heads, self.kv_heads, self.head_dim,
                             window=self.window, scale=self.scale)
        out = ctx.buffer("attn.out", (t, self.width), self.dtype)
        return self.k.linear(attn, self.o, out, defer=True)
