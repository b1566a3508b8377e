"""A single-GPU inference engine for the Llama-3 family on B200 (sm_100a).

    from iitj_llm_coopt_b200 import LLM, SamplingParams
    llm = LLM("path/to/model_dir", dtype="bfloat16")
    outs = llm.generate([[1, 2, 3]], SamplingParams(max_tokens=16))
"""
from .config import EngineConfig, LlamaConfig
from .engine import LLM, Engine, RequestOutput, Sequence, StaticPolicy, StepEntry, build_engine
from .sampling import SamplingParams

__all__ = ["LLM", "Engine", "EngineConfig", "LlamaConfig", "RequestOutput", "SamplingParams", "Sequence",
           "StaticPolicy", "StepEntry", "build_engine"]
