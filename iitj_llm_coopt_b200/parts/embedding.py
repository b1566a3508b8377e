"""Token embedding and the output head.

`Embedding`: x = table[token_ids] (engine/model.py:191), written as the float32 residual stream.
`OutputHead`: logits = x . W^T in float32 (engine/model.py:215-218); W is the embedding table
when the model ties them (engine/model.py:106).
"""
from __future__ import annotations

import torch

from .base import ParamSpec, Part


class Embedding(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype=None):
        self.spec, self.vocab, self.width, self.k, self.scale = spec, spec.vocab, spec.width, kernels, spec.scale
        self.weight = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.vocab, spec.width), kind="table")}

    def forward(self, ctx):
        out = ctx.buffer("residual", (ctx.num_tokens, self.width), torch.float32)
        return self.k.embed(ctx.token_ids, self.weight, out, self.scale)


class OutputHead(Part):
    graph_safe = True

    tied_parameter = "weight"     # the parameter that is the embedding's table when the model ties them

    def __init__(self, spec, kernels, dtype=None):
        self.spec, self.vocab, self.width, self.k, self.scale = spec, spec.vocab, spec.width, kernels, spec.scale
        self.weight = None

    @classmethod
    def parameters(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.vocab, spec.width), kind="matrix")}

    def forward(self, ctx, x):
        logits = ctx.buffer("logits", (x.shape[0], self.vocab), torch.float32)
        self.k.linear(x, self.weight, logits)
        if self.scale != 1.0:
            self.k.scale_(logits, self.scale)
        return logits
