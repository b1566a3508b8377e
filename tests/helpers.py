"""Shared helpers of the tests: building engines on either device, replay drivers, comparisons."""
import torch

from iitj_llm_coopt_b200 import EngineConfig, build_engine
from iitj_llm_coopt_b200.engine import StepEntry


def make_engine(model_dir, dtype="float32", page_size=16, num_pages=64, device=None, **kw):
    """Engine on the GPU with the CUDA kernels, or (device='cpu') on the CPU with the plain-torch
    kernel double of tests/torch_kernels.py."""
    device = device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    kernels = None
    if device == "cpu":
        from torch_kernels import TorchKernels
        kernels = TorchKernels()
    ec = EngineConfig(dtype=dtype, page_size=page_size, num_pages=num_pages, device=device, **kw)
    return build_engine(model_dir, ec, kernels=kernels)


def rel_err(got, want):
    return (got.float().cpu() - want.float().cpu()).abs().max().item() / max(want.abs().max().item(), 1e-30)


def run_steps(engine, steps):
    """steps: list of (entries, ends) with entries = [(request, tokens, want)].  Returns
    {(request, position): logits row} for every wanted place."""
    runner, cache = engine.runner, engine.cache
    rows = {}
    for entries, ends in steps:
        es = []
        for rid, toks, want in entries:
            if not cache.has(rid):
                cache.admit(rid)
            es.append(StepEntry(rid, list(toks), list(want)))
        starts = [cache.num_tokens(e.request) for e in es]
        logits = runner.step(es)
        if logits is not None:
            logits = logits.float().cpu()
            r = 0
            for e, s in zip(es, starts):
                for w in e.want:
                    rows[(e.request, s + w)] = logits[r].clone()
                    r += 1
        for rid in ends:
            cache.release(rid)
    return rows
