from .engine import EngineConfig, canonical_dtype
from .errors import ConfigError
from .llama import LlamaConfig
from .registry import ARCHITECTURES, architecture_for, load_config, register_architecture
from .specs import (CacheNeed, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec,
                    NormSpec, PositionSpec)
