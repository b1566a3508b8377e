"""What one step hands to the model: the flattened batch on the device.

All index tensors are int32 views into one device buffer that was filled by a single
host-to-device copy (engine/runner.py).  The reference's `Batch` (engine/model.py:54-65)
carries the same fields; added here are `token_request` (which request of the step each
token belongs to), `state_slots`, `first_portion`, and one block table and slot mapping
per cache group.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class GroupMeta:
    """Per cache group: where this step's tokens are stored and where earlier ones lie."""
    block_table: torch.Tensor      # [B, W] int32, page ids (entries past a request's pages are 0)
    slots: torch.Tensor            # [T] int32, page * page_size + offset of each new token
    token_request: torch.Tensor    # [T] int32 (same tensor for all groups)
    positions: torch.Tensor        # [T] int32
    # host copies for kernels that plan their grid on the host
    query_lens: list = field(default_factory=list)
    seq_lens_host: list = field(default_factory=list)
    cu_seqlens: torch.Tensor | None = None
    seq_lens: torch.Tensor | None = None
    attention_plan: object = None  # kernels.AttentionPlan: decode items and prefill tiles of this step


class Workspace:
    """Named scratch tensors that live across steps, so a step allocates nothing once
    every buffer has reached its largest size."""

    def __init__(self, device):
        self.device = device
        self._flat: dict = {}
        self._views: dict = {}   # (name, dtype, shape) -> the view handed out last time (same storage, same shape)
        self.generation = 0      # bumped whenever a buffer is (re)allocated: captured graphs then hold stale addresses

    def get(self, name: str, shape, dtype) -> torch.Tensor:
        # every layer of every step asks for the same few (name, shape) pairs: the view is made once
        vkey = (name, dtype, shape if type(shape) is tuple else tuple(shape))
        view = self._views.get(vkey)
        if view is not None:
            return view
        view = self._make(name, vkey[2], dtype)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[vkey] = view
        return view

    def _make(self, name: str, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        flat = self._flat.get(key)
        if flat is None or flat.numel() < n:
            # grown to the next power of two (in steps of 64 Mi elements beyond that), so that a buffer whose
            # size creeps up step by step (one more logits row) is allocated a few times, not every step
            cap = 1 << max(n - 1, 0).bit_length() if n <= (1 << 26) else -(-n // (1 << 26)) * (1 << 26)
            flat = torch.empty(cap, dtype=dtype, device=self.device)
            self._flat[key] = flat
            self._views.clear()      # views of the old storage must not be handed out again
            self.generation += 1
        return flat[:n].view(*shape)


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    num_logits: int
    token_ids: torch.Tensor        # [T]
    positions: torch.Tensor        # [T]
    token_request: torch.Tensor    # [T]
    cu_seqlens: torch.Tensor       # [B+1] offsets of each request's new tokens
    seq_lens: torch.Tensor         # [B] stored + new tokens
    logit_rows: torch.Tensor       # [N] rows of the hidden states that want logits
    state_slots: torch.Tensor      # [B]
    first_portion: torch.Tensor    # [B] 1 where the request's tokens start at position 0
    groups: dict                   # group index -> GroupMeta
    cache: object                  # CacheManager
    workspace: Workspace
    # host-side copies, for parts that must loop over requests on the host
    requests: list = field(default_factory=list)
    query_lens: list = field(default_factory=list)
    starts: list = field(default_factory=list)
    slots_host: list = field(default_factory=list)
    shared: dict = field(default_factory=dict)   # per-step results that several layers share (e.g. rotary tables)
    prepared: dict = field(default_factory=dict)  # prepare_key -> the StepPlan a part made for this step (parts/base.py)

    def buffer(self, name: str, shape, dtype) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype)

    def group(self, index: int) -> GroupMeta:
        return self.groups[index]
