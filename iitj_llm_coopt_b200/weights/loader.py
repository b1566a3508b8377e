"""Reads a model folder's safetensors files into the parameters of the generic decoder.

Tensors are found by name (the architecture maps each parameter, and each piece of a
concatenated parameter, to a checkpoint tensor name).  Before anything is read, the
names and shapes of the whole checkpoint are compared with what the model needs; one
`WeightError` lists every missing tensor, every unexpected tensor and every wrong shape.

Precision rules:
  engine dtype float32   every parameter is converted to float32.
  engine dtype bfloat16  matrices and embedding tables are bfloat16 (a bfloat16 file is
                         used as stored); vectors (norm gains) keep a float32 stored type;
                         integer tensors become int32.
The reference loads every key and casts it to the model dtype without checks
(engine/model.py:139-142) and fuses q/k/v and gate/up by concatenation (113-116); the
fusion here writes each piece straight into its rows of the fused tensor.
"""
from __future__ import annotations

import glob
import os

import torch
from safetensors import safe_open

from ..models.decoder import model_parameter_specs

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
              "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
              "BOOL": torch.bool}


class WeightError(ValueError):
    def __init__(self, model_dir, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"weights in {model_dir!r} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} is {tuple(got)}, expected {tuple(want)}" for n, got, want in self.wrong_shape))
        lines.extend(f"  {o}" for o in other)
        super().__init__("\n".join(lines))


def checkpoint_index(model_dir: str) -> dict:
    """{tensor name: (file, shape, torch dtype)} over every *.safetensors file of the folder."""
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"{model_dir!r} holds no .safetensors file")
    index = {}
    for path in files:
        with safe_open(path, framework="pt", device="cpu") as f:
            for name in f.keys():
                sl = f.get_slice(name)
                index[name] = (path, tuple(sl.get_shape()), _ST_DTYPES.get(sl.get_dtype(), None))
    return index


def expected_tensors(arch, spec) -> dict:
    """{checkpoint name: (shape, parameter path, first row in the parameter)}"""
    want = {}
    for path, ps in model_parameter_specs(spec).items():
        if ps.pieces is None:
            want[arch.checkpoint_name(path, None)] = (tuple(ps.shape), path, 0)
        else:
            row = 0
            for piece, rows in ps.pieces:
                want[arch.checkpoint_name(path, piece)] = ((rows,) + tuple(ps.shape[1:]), path, row)
                row += rows
    return want


def target_dtype(kind: str, stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if kind == "vector" and stored == torch.float32:
        return torch.float32
    return engine_dtype


def load_parameters(model_dir: str, arch, config, spec, engine_dtype: torch.dtype, device="cuda") -> dict:
    index = checkpoint_index(model_dir)
    want = expected_tensors(arch, spec)
    missing = sorted(n for n in want if n not in index)
    unexpected = sorted(n for n in index if n not in want and not arch.is_ignored(n, config))
    wrong = [(n, index[n][1], want[n][0]) for n in sorted(want) if n in index and index[n][1] != want[n][0]]
    other = [f"{n}: storage type is not supported" for n in sorted(want) if n in index and index[n][2] is None]
    if missing or unexpected or wrong or other:
        raise WeightError(model_dir, missing, unexpected, wrong, other)

    pspecs = model_parameter_specs(spec)
    by_param: dict = {}
    for name, (shape, path, row) in want.items():
        by_param.setdefault(path, []).append((row, name, shape))
    params = {}
    handles = {}
    try:
        for path, pieces in by_param.items():
            ps = pspecs[path]
            stored = {index[n][2] for _, n, _ in pieces}
            dt = target_dtype(ps.kind, torch.float32 if torch.float32 in stored else next(iter(stored)), engine_dtype)
            full = torch.empty(ps.shape, dtype=dt, device=device)
            for row, name, shape in sorted(pieces):
                file = index[name][0]
                if file not in handles:
                    handles[file] = safe_open(file, framework="pt", device="cpu")
                full[row:row + shape[0]].copy_(handles[file].get_tensor(name))
            params[path] = full
    finally:
        handles.clear()
    return params
