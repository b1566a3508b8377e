"""The generic decoder: embedding, the layers in their run order, final norm, output head.

It is assembled from a `ModelSpec` alone.  Each layer's arrangement declares the names and
families of its parts; the parts are looked up in the registries by the `kind` of their spec
record, so different layers of one model can have different arrangements, mixers and
feed-forwards; embedding and head come from registries too; the run order (`spec.order`) is
walked as data.
Forward formulas in the reference's order: engine/model.py:181-213.
"""
from __future__ import annotations

import torch

from .. import parts as P
from ..parts.base import delta_for


def _lookup(family: str, spec, what: str):
    registry = P.FAMILIES[family]
    if spec.kind not in registry:
        raise KeyError(f"{what} kind {spec.kind!r} is not registered; known: {', '.join(sorted(registry))}")
    return registry[spec.kind]


def _arrangement(layer):
    if layer.arrangement not in P.ARRANGEMENTS:
        raise KeyError(f"arrangement {layer.arrangement!r} is not registered; known: {', '.join(sorted(P.ARRANGEMENTS))}")
    return P.ARRANGEMENTS[layer.arrangement]


def layer_parts(layer) -> list:
    """[(part name, family, spec record, class)] of a layer, in the order its arrangement declares them."""
    arr = _arrangement(layer)
    names = set(layer.names())
    if names != set(arr.PARTS):
        raise KeyError(f"arrangement {layer.arrangement!r} is wired from {sorted(arr.PARTS)}, the layer gives {sorted(names)}")
    if sum(1 for f in arr.PARTS.values() if f == "mixer") > 1:
        raise ValueError(f"arrangement {layer.arrangement!r} declares more than one mixer (one cache entry per call)")
    return [(name, family, layer.part(name), _lookup(family, layer.part(name), name)) for name, family in arr.PARTS.items()]


def model_parameter_specs(spec) -> dict:
    """{parameter path: ParamSpec} of the whole model, without building anything."""
    emb = spec.embedding_spec()
    out = {f"embedding.{n}": ps for n, ps in _lookup("embedding", emb, "embedding").parameters(emb).items()}
    for i, layer in enumerate(spec.layers):
        for part_name, _family, part_spec, cls in layer_parts(layer):
            for pname, pspec in cls.parameters(part_spec).items():
                out[f"layers.{i}.{part_name}.{pname}"] = pspec
    for pname, pspec in _lookup("norm", spec.final_norm, "norm").parameters(spec.final_norm).items():
        out[f"final_norm.{pname}"] = pspec
    head = spec.head_spec()
    head_cls = _lookup("head", head, "head")
    for pname, pspec in head_cls.parameters(head).items():
        if spec.tie_embeddings and pname == getattr(head_cls, "tied_parameter", None):
            continue                      # the embedding's table stands in
        out[f"lm_head.{pname}"] = pspec
    return out


def cache_needs(spec) -> list:
    """One CacheNeed per cache entry (indexed by LayerCall.cache of the writing call)."""
    from ..config.specs import CacheNeed
    entries = {}
    for call in spec.order:
        need = CacheNeed()
        for _name, family, part_spec, cls in layer_parts(spec.layers[call.layer]):
            if family == "mixer":
                need = cls.cache_need(part_spec)
        if call.write:
            if call.cache in entries and entries[call.cache] != need:
                raise ValueError(f"cache entry {call.cache} is written by layers with different needs")
            entries[call.cache] = need
    for call in spec.order:
        if call.cache not in entries:
            raise ValueError(f"run order reads cache entry {call.cache} that no call writes")
    n = max(entries) + 1 if entries else 0
    return [entries.get(i, CacheNeed()) for i in range(n)]


def build_part(family: str, part_spec, cls, kernels, dtype, device, name: str = ""):
    """One part from its spec record.  A mixer is handed its position encoding, built from the spec's `position`.
    `name` (the part's name in its arrangement) becomes `part.part_name`: parts that keep an output buffer in the
    step's workspace name it after that, so that two parts of one class in one layer do not share a buffer."""
    if family == "mixer":
        pos = None
        if getattr(part_spec, "position", None) is not None:
            pos_cls = _lookup("position", part_spec.position, "position encoding")
            pos = pos_cls(part_spec.position, kernels, dtype, device)
        part = cls(part_spec, kernels, dtype, position=pos)
    else:
        part = cls(part_spec, kernels, dtype)
    part.part_name = name
    return part


class DecoderModel:
    def __init__(self, spec, kernels, dtype, device="cuda"):
        self.spec, self.k, self.dtype, self.device = spec, kernels, dtype, device
        emb = spec.embedding_spec()
        self.embedding = build_part("embedding", emb, _lookup("embedding", emb, "embedding"), kernels, dtype, device)
        self.layers = []
        for layer in spec.layers:
            built = {name: build_part(family, part_spec, cls, kernels, dtype, device, name)
                     for name, family, part_spec, cls in layer_parts(layer)}
            self.layers.append(_arrangement(layer)(**built))
        self.final_norm = build_part("norm", spec.final_norm, _lookup("norm", spec.final_norm, "norm"), kernels, dtype, device,
                                     "final_norm")
        head = spec.head_spec()
        self.head = build_part("head", head, _lookup("head", head, "head"), kernels, dtype, device)

    def all_parts(self) -> list:
        """Every part of the model, the parts that parts own included (each object once)."""
        seen, out = set(), []
        for part in [self.embedding] + [p for b in self.layers for p in b.all_parts()] + [self.final_norm, self.head]:
            if id(part) not in seen:
                seen.add(id(part))
                out.append(part)
        return out

    @property
    def graph_safe(self) -> bool:
        """True if every part only launches shape-determined work, so decode steps can be captured."""
        return all(getattr(p, "graph_safe", False) for p in self.all_parts())

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
        head_params = dict(per_part.get("lm_head", {}))
        tied = getattr(self.head, "tied_parameter", None)
        if self.spec.tie_embeddings and tied is not None:
            head_params[tied] = per_part["embedding"][tied]       # the head reads the embedding's table (engine/model.py:106)
        self.head.load(head_params)
        for i, block in enumerate(self.layers):
            for part_name, part in block.parts().items():
                part.load(per_part.get(f"layers.{i}.{part_name}", {}))

    def parameter_bytes(self) -> int:
        seen, total = set(), 0
        for part in self.all_parts():
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
