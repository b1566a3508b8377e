"""The generic decoder: embedding, the layers in their run order, final norm, output head.

It is assembled from a `ModelSpec` alone.  Each layer's parts are looked up in the part
registries by the `kind` of their spec record, so different layers of one model can have
different mixers and feed-forwards; the run order (`spec.order`) is walked as data.
Forward formulas in the reference's order: engine/model.py:181-213.
"""
from __future__ import annotations

import torch

from .. import parts as P
from ..parts.base import delta_for


def _layer_part_classes(layer):
    return {
        "mixer_norm": (P.NORMS, layer.mixer_norm),
        "mixer": (P.MIXERS, layer.mixer),
        "feed_forward_norm": (P.NORMS, layer.feed_forward_norm),
        "feed_forward": (P.FEED_FORWARDS, layer.feed_forward),
    }


def _lookup(registry, spec, what):
    if spec.kind not in registry:
        raise KeyError(f"{what} kind {spec.kind!r} is not registered; known: {', '.join(sorted(registry))}")
    return registry[spec.kind]


def model_parameter_specs(spec) -> dict:
    """{parameter path: ParamSpec} of the whole model, without building anything."""
    out = {"embedding.weight": P.Embedding.parameters(spec)["weight"]}
    for i, layer in enumerate(spec.layers):
        for part_name, (registry, part_spec) in _layer_part_classes(layer).items():
            cls = _lookup(registry, part_spec, part_name)
            for pname, pspec in cls.parameters(part_spec).items():
                out[f"layers.{i}.{part_name}.{pname}"] = pspec
    for pname, pspec in _lookup(P.NORMS, spec.final_norm, "norm").parameters(spec.final_norm).items():
        out[f"final_norm.{pname}"] = pspec
    if not spec.tie_embeddings:
        out["lm_head.weight"] = P.OutputHead.parameters(spec)["weight"]
    return out


def cache_needs(spec) -> list:
    """One CacheNeed per cache entry (indexed by LayerCall.cache of the writing call)."""
    entries = {}
    for call in spec.order:
        layer = spec.layers[call.layer]
        need = _lookup(P.MIXERS, layer.mixer, "mixer").cache_need(layer.mixer)
        if call.write:
            if call.cache in entries and entries[call.cache] != need:
                raise ValueError(f"cache entry {call.cache} is written by layers with different needs")
            entries[call.cache] = need
    for call in spec.order:
        if call.cache not in entries:
            raise ValueError(f"run order reads cache entry {call.cache} that no call writes")
    n = max(entries) + 1 if entries else 0
    from ..config.specs import CacheNeed
    return [entries.get(i, CacheNeed()) for i in range(n)]


class DecoderModel:
    def __init__(self, spec, kernels, dtype, device="cuda"):
        self.spec, self.k, self.dtype, self.device = spec, kernels, dtype, device
        self.embedding = P.Embedding(spec.vocab, spec.width, kernels, spec.embedding_scale)
        self.layers = []
        for layer in spec.layers:
            built = {}
            for part_name, (registry, part_spec) in _layer_part_classes(layer).items():
                cls = _lookup(registry, part_spec, part_name)
                if part_name == "mixer":
                    pos = None
                    if part_spec.position is not None:
                        pos_cls = _lookup(P.POSITION_ENCODINGS, part_spec.position, "position encoding")
                        pos = pos_cls(part_spec.position, kernels, dtype, device)
                    built[part_name] = cls(part_spec, kernels, dtype, position=pos)
                else:
                    built[part_name] = cls(part_spec, kernels, dtype)
            if layer.arrangement not in P.ARRANGEMENTS:
                raise KeyError(f"arrangement {layer.arrangement!r} is not registered")
            self.layers.append(P.ARRANGEMENTS[layer.arrangement](**built))
        self.final_norm = _lookup(P.NORMS, spec.final_norm, "norm")(spec.final_norm, kernels, dtype)
        self.head = P.OutputHead(spec.vocab, spec.width, kernels, spec.logit_scale)

    @property
    def graph_safe(self) -> bool:
        """True if every part only launches shape-determined work, so decode steps can be captured."""
        mixers_ok = all(getattr(b.mixer.position, "graph_safe", True) for b in self.layers
                        if getattr(b.mixer, "position", None) is not None)
        return mixers_ok and all(getattr(b, "graph_safe", False) for b in self.layers) and \
            self.embedding.graph_safe and self.final_norm.graph_safe and self.head.graph_safe

    # ---- parameters ----------------------------------------------------------------------
    def load_parameters(self, params: dict) -> None:
        """`params`: {path: tensor} for every path of model_parameter_specs(spec)."""
        want = set(model_parameter_specs(self.spec))
        if set(params) != want:
            raise KeyError(f"parameters differ from the model's: missing {sorted(want - set(params))}, "
                           f"unexpected {sorted(set(params) - want)}")
        per_part: dict = {}
        for path, t in params.items():
            owner, name = path.rsplit(".", 1)
            per_part.setdefault(owner, {})[name] = t
        self.embedding.load(per_part["embedding"])
        self.final_norm.load(per_part["final_norm"])
        self.head.load(per_part["lm_head"] if not self.spec.tie_embeddings
                       else {"weight": per_part["embedding"]["weight"]})
        for i, block in enumerate(self.layers):
            for part_name, part in block.parts().items():
                part.load(per_part.get(f"layers.{i}.{part_name}", {}))

    def parameter_bytes(self) -> int:
        seen, total = set(), 0
        for part in [self.embedding, self.final_norm, self.head] + \
                [p for b in self.layers for p in b.parts().values()]:
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    # ---- forward -------------------------------------------------------------------------
    def forward(self, ctx):
        """Runs the tokens of `ctx` through the model; returns float32 logits [ctx.num_logits, vocab]
        for the rows in ctx.logit_rows (None if no row is wanted)."""
        residual, delta = self.embedding.forward(ctx), None
        for call in self.spec.order:
            residual, delta = self.layers[call.layer].forward(ctx, residual, delta, call)
        if ctx.num_logits == 0:
            return None
        x = self.final_norm.forward(ctx, residual, delta_for(self.final_norm, delta), rows=ctx.logit_rows)
        return self.head.forward(ctx, x)


def build_model(spec, kernels, dtype, device="cuda") -> DecoderModel:
    return DecoderModel(spec, kernels, dtype, device)
