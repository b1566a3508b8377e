"""The part registries: a layer's spec names its parts by these keys.

Adding a part means writing a class with the interface described in parts/base.py and
registering it here (or from outside with the `register_*` functions); the model
builder (models/decoder.py) looks the classes up by the `kind` of each spec record.
"""
from __future__ import annotations

from .base import ParamSpec, Part
from .block import PreNormBlock
from .embedding import Embedding, OutputHead
from .feed_forward import SwiGLU
from .mixer import PagedAttention
from .norm import RMSNorm
from .position import NoPosition, RotaryEmbedding, rope_inverse_frequencies

NORMS = {"rmsnorm": RMSNorm}
POSITION_ENCODINGS = {"rope": RotaryEmbedding, "none": NoPosition}
MIXERS = {"attention": PagedAttention}
FEED_FORWARDS = {"swiglu": SwiGLU}
ARRANGEMENTS = {"prenorm": PreNormBlock}


def register_norm(kind, cls):
    NORMS[kind] = cls


def register_position_encoding(kind, cls):
    POSITION_ENCODINGS[kind] = cls


def register_mixer(kind, cls):
    MIXERS[kind] = cls


def register_feed_forward(kind, cls):
    FEED_FORWARDS[kind] = cls


def register_arrangement(kind, cls):
    ARRANGEMENTS[kind] = cls
