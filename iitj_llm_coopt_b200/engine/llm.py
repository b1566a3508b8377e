"""The Python entry point: build an engine from a model folder and generate.

The reference has no class of this name; its in-process use is "build Engine, append
Sequences to scheduler.waiting, loop engine.step() until finished, read
seq.tokens[prompt_len:]" (tests/elastic_check.py:24-38, eval/quality.py:75-84).  `LLM.generate`
is that loop.  Token ids go in and come out; no tokenizer is involved.  Options carry the
reference's names (engine/server.py:188-196; engine/engine.py:159-162).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch

from ..cache import CacheManager
from ..config import EngineConfig, load_config
from ..models.decoder import build_model, cache_needs
from ..sampling import Sampler, SamplingParams
from ..weights import load_parameters, random_parameters
from .engine import Engine
from .policy import StaticPolicy
from .runner import ModelRunner

TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: list
    token_ids: list
    finish_reason: str | None
    ttft: float | None = None          # seconds from submission to the first token
    e2e: float | None = None           # seconds from submission to the end
    num_preemptions: int = 0


def workspace_bytes_estimate(spec, tokens: int, rows: int, itemsize: int) -> int:
    """Rough size of the step's scratch tensors for `tokens` tokens and `rows` logits rows (twice what the
    shapes need: the workspace grows its buffers to powers of two)."""
    widest = 0
    for layer in spec.layers:
        cols = 3 * spec.width
        for _name, ps in layer.parts:        # whatever sizes the layer's parts name: projections, inner widths
            heads, kv_heads, head_dim = (getattr(ps, a, 0) or 0 for a in ("heads", "kv_heads", "head_dim"))
            cols += (2 * heads + 2 * kv_heads) * head_dim + 3 * (getattr(ps, "inner", 0) or 0)
        widest = max(widest, cols)
    return 2 * (tokens * (widest * itemsize + 4 * spec.width) + rows * spec.vocab * 4) + (64 << 20)


def build_engine(model: str | None = None, engine_config: EngineConfig | None = None, *, config=None,
                 architecture=None, random_seed: int | None = None, kernels=None, policy=None) -> Engine:
    """Engine for the model folder `model`, or for a typed `config` with random weights
    drawn on the device from `random_seed` (no files)."""
    ec = engine_config or EngineConfig()
    dtype = TORCH_DTYPE[ec.dtype]
    if kernels is None:
        from .. import kernels as _k
        kernels = _k.load()
    if model is not None:
        arch, cfg = load_config(model)
    else:
        if config is None:
            raise ValueError("give a model folder or a config")
        from ..config.registry import architecture_for
        arch = architecture or architecture_for(config.to_dict())
        cfg = config
    spec = arch.model_spec(cfg)
    device = torch.device(ec.device)
    with torch.cuda.device(device) if device.type == "cuda" else _null():
        net = build_model(spec, kernels, dtype, device)
        if model is not None:
            params = load_parameters(model, arch, cfg, spec, dtype, device)
        else:
            params = random_parameters(arch, spec, random_seed or 0, dtype, device=device)
        net.load_parameters(params)
        del params
        needs = cache_needs(spec)
        itemsize = 2 if dtype == torch.bfloat16 else 4
        step_tokens = ec.max_num_batched_tokens

        def pages_that_fit(budget_bytes):
            return CacheManager.pages_for_bytes(needs, ec.page_size, budget_bytes, itemsize, ec.max_num_seqs, step_tokens)
        if ec.num_pages is not None:
            num_pages = ec.num_pages
        elif ec.kv_gb is not None:
            num_pages = pages_that_fit(ec.kv_gb * 2**30)
        else:
            # what is left under the utilisation cap after the weights, the step's scratch tensors and a margin
            # (engine/engine.py:174-192 measures the activations instead of estimating them)
            free, total = torch.cuda.mem_get_info(device)
            work = workspace_bytes_estimate(spec, ec.max_num_batched_tokens, ec.max_num_seqs, itemsize)
            num_pages = pages_that_fit(total * ec.gpu_memory_utilization - (total - free) - work - (256 << 20))
            # no need for more pages than max_num_seqs full-length requests could ever fill
            num_pages = min(num_pages, ec.max_num_seqs * (-(-ec.max_model_len // ec.page_size)))
        if num_pages <= 0:
            raise RuntimeError("no memory left for the key/value cache")
        cache = CacheManager(needs, ec.page_size, num_pages, max_requests=ec.max_num_seqs, dtype=dtype, device=device,
                             max_step_tokens=step_tokens)
        runner = ModelRunner(net, cache, device, cuda_graphs=ec.cuda_graphs)
        sampler = Sampler(kernels, ec.seed, device)
    pol = policy or StaticPolicy(max_num_seqs=ec.max_num_seqs, max_batched_tokens=ec.max_num_batched_tokens,
                                 watermark=ec.watermark)
    eng = Engine(runner, cache, sampler, pol, max_model_len=min(ec.max_model_len, spec.max_position),
                 eos_ids=spec.eos_token_ids, lookahead=ec.lookahead and device.type == "cuda")
    eng.model_config, eng.model_spec, eng.engine_config = cfg, spec, ec
    return eng


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class LLM:
    def __init__(self, model: str | None = None, dtype: str = "bfloat16", *, config=None, random_seed=None,
                 page_size: int = 16, num_pages: int | None = None, kv_gb: float | None = None,
                 gpu_memory_utilization: float = 0.9, max_model_len: int = 32768, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 2048, seed: int = 0, device: str = "cuda:0", kernels=None,
                 cuda_graphs: bool = True, lookahead: bool = True):
        ec = EngineConfig(dtype=dtype, page_size=page_size, num_pages=num_pages, kv_gb=kv_gb,
                          gpu_memory_utilization=gpu_memory_utilization, max_model_len=max_model_len,
                          max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens, seed=seed,
                          device=device, cuda_graphs=cuda_graphs, lookahead=lookahead)
        self.engine = build_engine(model, ec, config=config, random_seed=random_seed, kernels=kernels)

    def generate(self, prompt_token_ids, sampling_params=None, on_output=None) -> list:
        """prompt_token_ids: a list of prompts (each a list of token ids).  sampling_params:
        one SamplingParams for all, or one per prompt.  `on_output(sequence, new_token_ids, finished)` is
        called as tokens arrive, as the reference's Sequence.on_output (engine/engine.py:40, 483-484).
        Returns RequestOutputs in order."""
        if prompt_token_ids and isinstance(prompt_token_ids[0], int):
            prompt_token_ids = [prompt_token_ids]
        n = len(prompt_token_ids)
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * n
        if len(sampling_params) != n:
            raise ValueError("one SamplingParams per prompt, or one for all")
        t0 = time.perf_counter()
        seqs = [self.engine.new_sequence(p, sp.max_tokens, sp.temperature, sp.ignore_eos, sp.seed, on_output)
                for p, sp in zip(prompt_token_ids, sampling_params)]
        self.engine.run_until_done()
        return [RequestOutput(request_id=s.seq_id, prompt_token_ids=s.tokens[:s.prompt_len],
                              token_ids=s.tokens[s.prompt_len:], finish_reason=s.finish_reason,
                              ttft=(s.first_token_time - t0) if s.first_token_time else None,
                              e2e=(s.finish_time - t0) if s.finish_time else None,
                              num_preemptions=s.num_preemptions) for s in seqs]
