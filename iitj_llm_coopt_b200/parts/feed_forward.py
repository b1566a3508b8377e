"""Feed-forward parts.

`SwiGLU`: x -> (silu(x Wgate^T) * (x Wup^T)) Wdown^T, no bias (engine/model.py:210-211), with
gate and up stored as one [2*inner, width] matrix, gate rows first (engine/model.py:116).
"""
from __future__ import annotations

from .base import ParamSpec, Part


class SwiGLU(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype):
        if spec.activation != "silu":
            raise ValueError(f"SwiGLU: activation {spec.activation!r} is not supported")
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.inner = spec.width, spec.inner
        self.gate_up = self.down = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {
            "gate_up": ParamSpec((2 * spec.inner, spec.width), pieces=(("gate", spec.inner), ("up", spec.inner))),
            "down": ParamSpec((spec.width, spec.inner)),
        }

    def forward(self, ctx, x):
        t = x.shape[0]
        act = ctx.buffer("ffn.act", (t, self.inner), self.dtype)
        self.k.linear(x, self.gate_up, act, swiglu=True)
        out = ctx.buffer("ffn.out", (t, self.width), self.dtype)
        return self.k.linear(act, self.down, out, defer=True)
