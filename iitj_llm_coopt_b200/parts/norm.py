"""RMSNorm over the float32 residual stream.

y = x * rsqrt(mean(x^2) + eps) * weight  (engine/model.py:85-89), statistics in float32.
The reference's fused form `residual += x; x = norm(residual)` (engine/model.py:236, 249, 254)
is the `delta` argument here.
"""
from __future__ import annotations

from .base import ParamSpec, Part


class RMSNorm(Part):
    graph_safe = True
    takes_partial_sums = True     # `delta` may be the k-split parts of a matrix product: added while they are read

    def __init__(self, spec, kernels, dtype):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.eps = spec.width, spec.eps
        self.weight = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.width,), kind="vector")}

    def forward(self, ctx, residual, delta=None, rows=None):
        n = rows.shape[0] if rows is not None else residual.shape[0]
        out = ctx.buffer(f"norm.{self.part_name}.out" if rows is None else f"norm.{self.part_name}.rows", (n, self.width), self.dtype)
        return self.k.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows=rows)
