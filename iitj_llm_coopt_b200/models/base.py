"""What an architecture has to say for itself.

An `Architecture` is a small record in the registry (config/registry.py): the name that
config.json carries in "architectures", the typed configuration class that reads the
file's keys, and the rule that maps each parameter of the generic decoder
(models/decoder.py: "layers.3.mixer.qkv", piece "k", ...) to the checkpoint's tensor name.
Everything else (parts, cache, step function, scheduler) is shared by all architectures.

To add one: write its config class with `from_dict` and `model_spec()`, subclass
`Architecture` with `checkpoint_name`, and call `register_architecture(MyArch())`.
"""
from __future__ import annotations

import fnmatch


class Architecture:
    name: str = ""
    config_class = None
    ignored_tensors: tuple = ()      # fnmatch patterns of checkpoint tensors that may be present and are unused

    def model_spec(self, config):
        return config.model_spec()

    def checkpoint_name(self, path: str, piece: str | None) -> str:
        """Checkpoint tensor name for parameter `path` (and piece of a concatenated tensor)."""
        raise NotImplementedError

    def is_ignored(self, tensor_name: str, config) -> bool:
        return any(fnmatch.fnmatch(tensor_name, p) for p in self.ignored_tensors)
