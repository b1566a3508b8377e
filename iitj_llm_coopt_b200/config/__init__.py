from .engine import EngineConfig, canonical_dtype
from .llama import ConfigError, LlamaConfig
from .registry import ARCHITECTURES, architecture_for, load_config, register_architecture
from .specs import (CacheNeed, FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec,
                    NormSpec, PositionSpec)
