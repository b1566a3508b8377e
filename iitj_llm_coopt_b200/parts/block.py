"""How the parts of one layer are wired.

`PreNormBlock` (the reference's decoder layer, engine/model.py:192-211 and its fused form
230-253): the residual stream stays apart in float32; every sub-layer's output is a
`delta` that the next norm adds into the residual before normalising:

    x = mixer_norm(residual += delta_in);        a = mixer(x)
    x = feed_forward_norm(residual += a);        delta_out = feed_forward(x)
"""
from __future__ import annotations

from .base import delta_for


class PreNormBlock:
    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts().values())

    def parts(self) -> dict:
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "feed_forward_norm": self.feed_forward_norm, "feed_forward": self.feed_forward}

    def forward(self, ctx, residual, delta, call):
        x = self.mixer_norm.forward(ctx, residual, delta_for(self.mixer_norm, delta))
        a = self.mixer.forward(ctx, x, call)
        x = self.feed_forward_norm.forward(ctx, residual, delta_for(self.feed_forward_norm, a))
        return residual, self.feed_forward.forward(ctx, x)
