"""Turns logits rows into token ids with the sampling kernel.

Greedy rows take the argmax (engine/spec_decode.py:14-15; the lowest index wins ties, as
torch.argmax does).  Rows with temperature T > 0 are drawn from softmax(logits / T)
(engine/spec_decode.py:16-17) by the Gumbel-max identity; the random stream of a row is
keyed by (engine seed, request seed, index of the token in its request), so a request's
tokens do not depend on batching.  One device-to-host copy per call brings the ids back.
"""
from __future__ import annotations

import torch

_MASK = (1 << 64) - 1


def mix64(z: int) -> int:
    """splitmix64 finaliser on Python ints (the kernel's mix64)."""
    z &= _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def row_key(engine_seed: int, request_seed: int, token_index: int) -> int:
    """64-bit key of one sampled token."""
    k = mix64(engine_seed + 0x9E3779B97F4A7C15)
    k = mix64(k ^ mix64(request_seed + 0xD1B54A32D192ED03))
    return mix64(k ^ mix64(token_index + 0x8CB92BA72F3D8DD7))


def _signed(u: int) -> int:
    return u - (1 << 64) if u >= (1 << 63) else u


class Sampler:
    def __init__(self, kernels, seed: int = 0, device="cuda"):
        self.k, self.seed, self.device = kernels, seed, device
        self._out = None
        self._host = None

    def _buffers(self, n):
        if self._out is None or self._out.numel() < n:
            cap = max(256, 2 * n)
            self._out = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._host = torch.empty(cap, dtype=torch.int32)
            if torch.cuda.is_available():
                self._host = self._host.pin_memory()
        return self._out[:n], self._host[:n]

    def sample(self, logits, rows: list) -> list:
        """rows[i] = (temperature, request seed, token index) for logits row i; returns ids."""
        n = logits.shape[0]
        if n != len(rows):
            raise ValueError(f"{n} logits rows but {len(rows)} sampling records")
        out, host = self._buffers(n)
        if all(t <= 0 for t, _, _ in rows):
            self.k.sample(logits, None, None, out)
        else:
            temps = torch.tensor([float(t) for t, _, _ in rows], dtype=torch.float32)
            keys = torch.tensor([_signed(row_key(self.seed, s, i)) for _, s, i in rows], dtype=torch.int64)
            self.k.sample(logits, temps.to(self.device), keys.to(self.device), out)
        host.copy_(out)          # synchronous: the step's one device-to-host read
        return host.tolist()
