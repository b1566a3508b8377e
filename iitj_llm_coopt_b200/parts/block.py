"""How the parts of one layer are wired.

An arrangement declares, in `PARTS`, the names of its parts and the family each is looked up in ("norm", "mixer",
"feed_forward": parts.FAMILIES); a `LayerSpec` holds one spec record per name, the model builder builds the parts and
hands them over as keywords.  At most one part of an arrangement is of family "mixer": it owns the layer's cache
entry.  `forward(ctx, residual, delta, call)` returns the new (residual, delta): the residual stream stays apart in
float32, and a sub-layer's output travels as a `delta` that the next norm adds into the residual before it normalises.

`PreNormBlock` (the reference's decoder layer, engine/model.py:192-211 and its fused form 230-253):

    x = mixer_norm(residual += delta_in);        a = mixer(x)
    x = feed_forward_norm(residual += a);        delta_out = feed_forward(x)
"""
from __future__ import annotations

from .base import delta_for


class Arrangement:
    PARTS: dict = {}             # part name -> family

    def __init__(self, **parts):
        missing = [n for n in self.PARTS if n not in parts]
        extra = [n for n in parts if n not in self.PARTS]
        if missing or extra:
            raise TypeError(f"{type(self).__name__} is wired from {sorted(self.PARTS)}; missing {missing}, unexpected {extra}")
        self._parts = dict(parts)
        for name, part in parts.items():
            setattr(self, name, part)

    def parts(self) -> dict:
        return self._parts

    def all_parts(self) -> list:
        """The parts and the parts they own (a mixer's position encoding)."""
        out = []
        for p in self._parts.values():
            out.append(p)
            out.extend(getattr(p, "subparts", lambda: ())())
        return out

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.all_parts())

    def forward(self, ctx, residual, delta, call):
        raise NotImplementedError


class PreNormBlock(Arrangement):
    PARTS = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, ctx, residual, delta, call):
        x = self.mixer_norm.forward(ctx, residual, delta_for(self.mixer_norm, delta))
        a = self.mixer.forward(ctx, x, call)
        x = self.feed_forward_norm.forward(ctx, residual, delta_for(self.feed_forward_norm, a))
        return residual, self.feed_forward.forward(ctx, x)
