"""The one registry from an architecture's name (config.json "architectures"[0]) to its model.

The reference hard-wires `Llama.from_pretrained` (engine/engine.py:168-169); here the name in
config.json picks an `Architecture` record: the typed configuration class that reads the
file's keys, and the rules that turn checkpoint tensor names into the parts' parameters.
"""
from __future__ import annotations

import json
import os

from .errors import ConfigError

ARCHITECTURES: dict = {}


def register_architecture(arch) -> None:
    """`arch` is an instance of models.base.Architecture; its `name` is the registry key."""
    ARCHITECTURES[arch.name] = arch


def architecture_for(config_dict: dict):
    _ensure_builtin()
    names = config_dict.get("architectures") or []
    if not names:
        raise ConfigError("config.json lacks 'architectures'; known: " + ", ".join(sorted(ARCHITECTURES)))
    name = names[0]
    if name not in ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; known: "
                          + ", ".join(sorted(ARCHITECTURES)))
    return ARCHITECTURES[name]


def load_config(model_dir: str):
    """(architecture, typed config) for a model folder."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir!r} has no config.json")
    with open(path, encoding="utf-8") as f:
        raw = json.load(f)
    arch = architecture_for(raw)
    return arch, arch.config_class.from_dict(raw)


def _ensure_builtin() -> None:
    if not ARCHITECTURES:
        from ..models import llama  # noqa: F401  (registers itself)
