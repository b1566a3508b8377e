"""The part registries: a spec record names its part by `kind`, a registry per family of parts maps the kind to
the class.

Adding a part means writing a class with the interface described in parts/base.py and registering it here (or
from outside with the `register_*` functions); the model builder (models/decoder.py) looks the classes up by the
family an arrangement declares for each of its part names and by the `kind` of the part's spec record.
"""
from __future__ import annotations

from .base import ParamSpec, Part, StepPlan, StepShape
from .block import Arrangement, PreNormBlock
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
EMBEDDINGS = {"table": Embedding}
HEADS = {"linear": OutputHead}

# family name (what an arrangement's PARTS declares for a part name) -> registry
FAMILIES = {"norm": NORMS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS, "position": POSITION_ENCODINGS,
            "embedding": EMBEDDINGS, "head": HEADS}


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


def register_embedding(kind, cls):
    EMBEDDINGS[kind] = cls


def register_head(kind, cls):
    HEADS[kind] = cls
