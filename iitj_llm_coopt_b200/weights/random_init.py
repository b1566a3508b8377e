"""Seeded random weights, either straight into parameters or as a model folder on disk.

Matrices and embedding tables are N(0, std) and norm gains 1 + U(-0.1, 0.1), each tensor
from a generator seeded by (seed, tensor name), so a tensor's values do not depend on
which other tensors exist.  `write_model_dir` writes config.json and model.safetensors
under the checkpoint names of the architecture, so the loader's path is exercised by
every test that uses it.  (The reference has no random-weights mode.)
"""
from __future__ import annotations

import hashlib
import json
import os

import torch
from safetensors.torch import save_file

from ..config.registry import architecture_for
from ..weights.loader import expected_tensors
from ..models.decoder import model_parameter_specs


def _seed_for(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & (2**63 - 1)


def _draw(kind: str, shape, seed: int, name: str, std: float, device) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(_seed_for(seed, name))
    if kind == "vector":
        return 1.0 + (torch.rand(shape, generator=g, device=device, dtype=torch.float32) * 0.2 - 0.1)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std


def random_checkpoint(arch, spec, seed: int, dtype=torch.bfloat16, std: float = 0.02, device="cpu") -> dict:
    """{checkpoint tensor name: tensor} with the architecture's own names and shapes."""
    pspecs = model_parameter_specs(spec)
    out = {}
    for name, (shape, path, _row) in expected_tensors(arch, spec).items():
        out[name] = _draw(pspecs[path].kind, shape, seed, name, std, device).to(dtype).contiguous()
    return out


def random_parameters(arch, spec, seed: int, engine_dtype: torch.dtype, std: float = 0.02, device="cuda") -> dict:
    """Parameters of the generic decoder drawn on `device` (no file; for benchmarks).

    Values are drawn in float32 and rounded to bfloat16 first, as a bfloat16 checkpoint
    would hold them, so both engine precisions see the same numbers."""
    pspecs = model_parameter_specs(spec)
    params = {}
    for name, (shape, path, row) in expected_tensors(arch, spec).items():
        ps = pspecs[path]
        if path not in params:
            params[path] = torch.empty(ps.shape, dtype=engine_dtype, device=device)
        piece = _draw(ps.kind, shape, seed, name, std, device).to(torch.bfloat16)
        params[path][row:row + shape[0]].copy_(piece)
        del piece
    return params


def write_model_dir(config, out_dir: str, seed: int, dtype=torch.bfloat16, std: float = 0.02, device="cpu") -> str:
    """Writes `out_dir/config.json` and `out_dir/model.safetensors`; `config` is a typed
    configuration or a plain dict of config.json keys (with "architectures").  `device`: where the
    values are drawn (a GPU draws a large model in seconds; its generator gives other values than the CPU's)."""
    raw = config if isinstance(config, dict) else config.to_dict()
    arch = architecture_for(raw)
    typed = arch.config_class.from_dict(raw)
    os.makedirs(out_dir, exist_ok=True)
    tensors = random_checkpoint(arch, arch.model_spec(typed), seed, dtype=dtype, std=std, device=device)
    tensors = {name: t.cpu() for name, t in tensors.items()}
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(typed.to_dict(), f, indent=1)
    return out_dir

