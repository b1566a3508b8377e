"""Options of the engine itself (not of a model).

Names and defaults follow the reference's server flags and policy knobs
(engine/server.py:188-196: --max-num-seqs 256, --max-num-batched-tokens 2048, --kv-gb,
--max-model-len 32768, --gpu-memory-utilization 0.9, --seed 0, --dtype; engine/policy.py:13-16:
watermark 0.01; engine/engine.py:159-162: block_size 16).
"""
from __future__ import annotations

from dataclasses import dataclass

DTYPE_ALIASES = {
    "bfloat16": "bfloat16", "bf16": "bfloat16",
    "float32": "float32", "fp32": "float32", "float": "float32",
}


def canonical_dtype(name) -> str:
    key = str(name).replace("torch.", "").lower()
    if key not in DTYPE_ALIASES:
        raise ValueError(f"dtype {name!r} is not supported: use bfloat16 or float32")
    return DTYPE_ALIASES[key]


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"
    page_size: int = 16                 # tokens per cache page ("block_size" in the reference)
    num_pages: int | None = None        # explicit pool size, else from kv_gb, else from free memory
    kv_gb: float | None = None
    gpu_memory_utilization: float = 0.9
    max_model_len: int = 32768
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 2048
    watermark: float = 0.01             # fraction of pages kept free when admitting
    seed: int = 0
    cuda_graphs: bool = True            # replay decode-only steps from captured graphs
    lookahead: bool = True              # launch the next decode step before the host has read this one's tokens
    device: str = "cuda:0"

    def __post_init__(self):
        self.dtype = canonical_dtype(self.dtype)
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
