"""Errors of the configuration layer, shared by the registry and by every architecture's typed configuration."""
from __future__ import annotations


class ConfigError(ValueError):
    """A config.json that cannot be used: a key is missing, a value is out of range, an option is not supported,
    or the architecture is not registered."""
