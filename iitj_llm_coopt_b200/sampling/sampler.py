"""Turns logits rows into token ids with the sampling kernel.

Greedy rows take the argmax (engine/spec_decode.py:14-15; the lowest index wins ties, as
torch.argmax does).  Rows with temperature T > 0 are drawn from softmax(logits / T)
(engine/spec_decode.py:16-17) by the Gumbel-max identity; the random stream of a row is
keyed by (engine seed, request seed, index of the token in its request), so a request's
tokens do not depend on batching.  One device-to-host copy per call brings the ids back,
and with them the kernel library's health words (a kernel whose bounded wait ran out leaves a
code there): `fetch` raises instead of handing out tokens computed from such a kernel's output.
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


HEALTH = 4      # int32 entries in front of the ids: the library's health words


class _Slot:
    """Device output, pinned host copies and an event: one sampling call in flight.  The device output and its
    host copy hold the health words first, then the ids (one copy brings both)."""

    def __init__(self, cap, device):
        pin = torch.cuda.is_available()
        self.cap = cap
        self.both = torch.zeros(HEALTH + cap, dtype=torch.int32, device=device)
        self.health, self.out = self.both[:HEALTH], self.both[HEALTH:]
        self.temps = torch.empty(cap, dtype=torch.float32, device=device)
        self.keys = torch.empty(cap, dtype=torch.int64, device=device)
        self.host = torch.zeros(HEALTH + cap, dtype=torch.int32)
        self.temps_host = torch.empty(cap, dtype=torch.float32)
        self.keys_host = torch.empty(cap, dtype=torch.int64)
        if pin:
            self.host, self.temps_host, self.keys_host = self.host.pin_memory(), self.temps_host.pin_memory(), self.keys_host.pin_memory()
        self.event = torch.cuda.Event() if str(device).startswith("cuda") else None


class Sampler:
    """`launch` starts the kernel and the copy of the ids to pinned host memory and returns a handle;
    `fetch` waits for that copy.  Three slots rotate, so a step can be launched while the ids of the step
    before it are still on their way (and still feed that step's tokens on the device)."""

    def __init__(self, kernels, seed: int = 0, device="cuda"):
        self.k, self.seed, self.device = kernels, seed, device
        self._slots: list = [None, None, None]
        self._turn = 0

    def _slot(self, n):
        i = self._turn
        self._turn = (self._turn + 1) % len(self._slots)
        if self._slots[i] is None or self._slots[i].cap < n:
            self._slots[i] = _Slot(max(256, 2 * n), self.device)
        return self._slots[i]

    def _buffers(self, n):
        """(device ids, host ids) of a fresh slot (for callers that launch the kernel themselves)."""
        slot = self._slot(n)
        return slot.out[:n], slot.host[HEALTH:HEALTH + n]

    def launch(self, logits, rows: list):
        """rows[i] = (temperature, request seed, token index) for logits row i; returns a handle for `fetch`.
        `handle.ids` are the sampled ids on the device."""
        n = logits.shape[0]
        if n != len(rows):
            raise ValueError(f"{n} logits rows but {len(rows)} sampling records")
        slot = self._slot(n)
        out = slot.out[:n]
        if all(t <= 0 for t, _, _ in rows):
            self.k.sample(logits, None, None, out, health=slot.health)
        else:
            slot.temps_host[:n] = torch.tensor([float(t) for t, _, _ in rows], dtype=torch.float32)
            slot.keys_host[:n] = torch.tensor([_signed(row_key(self.seed, s, i)) for _, s, i in rows], dtype=torch.int64)
            slot.temps[:n].copy_(slot.temps_host[:n], non_blocking=True)
            slot.keys[:n].copy_(slot.keys_host[:n], non_blocking=True)
            self.k.sample(logits, slot.temps[:n], slot.keys[:n], out, health=slot.health)
        slot.host[:HEALTH + n].copy_(slot.both[:HEALTH + n], non_blocking=True)
        if slot.event is not None:
            slot.event.record()
        return _Handle(slot, n)

    def fetch(self, handle) -> list:
        if handle.slot.event is not None:
            handle.slot.event.synchronize()
        words = handle.slot.host[:HEALTH + handle.n].tolist()
        if any(words[:HEALTH]):
            self.k.check_health(words[:HEALTH])      # raises KernelError: these ids come from a kernel that gave up
        return words[HEALTH:]

    def sample(self, logits, rows: list) -> list:
        """Ids of the rows; one device-to-host read."""
        return self.fetch(self.launch(logits, rows))


class _Handle:
    def __init__(self, slot, n):
        self.slot, self.n = slot, n

    @property
    def ids(self):
        return self.slot.out[:self.n]
