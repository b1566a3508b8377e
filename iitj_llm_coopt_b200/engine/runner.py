"""The step function.

`ModelRunner.step(entries)` takes a batch of (request, its next tokens, the places among
them whose logits are wanted): portions of prompts beside single decoded tokens, cut
anywhere.  It runs only those tokens, as one flattened batch, on top of what earlier
steps left in the cache, stores their keys and values, and returns float32 logits at the
wanted places, in the order of the entries and of their `want` lists.

The flattening is the reference's build_batch (engine/batch.py:23-55): token ids,
positions, offsets of each request's tokens, lengths after the step, a padded block
table, the cache slot of every new token and the rows that need logits.  Differences:
all index arrays travel in one pinned buffer and one host-to-device copy; logits are
computed only where wanted (possibly nowhere); page tables are mirrored as arrays so a
decode step does not rebuild them from Python lists.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .context import GroupMeta, StepContext, Workspace


@dataclass
class StepEntry:
    request: object
    tokens: list
    want: list = field(default_factory=list)   # indices into `tokens`


class ModelRunner:
    def __init__(self, model, cache, device="cuda"):
        self.model, self.cache, self.device = model, cache, device
        self.vocab = model.spec.vocab
        self.workspace = Workspace(device)
        self._pinned = None          # int32 staging buffer (host, pinned)
        self._meta = None            # int32 device buffer the step's index arrays live in
        self._mirror: dict = {}      # (group, request) -> [np.int32 array, filled, the table it mirrors]
        self._copied = None          # event: the last host-to-device copy of the staging buffer is done
        self.steps = 0

    # ---- page-table mirror -----------------------------------------------------------
    def _table_row(self, group: int, request) -> np.ndarray:
        table = self.cache.table(group, request)
        n = len(table)
        rec = self._mirror.get((group, request))
        if rec is None or rec[2] is not table:
            rec = [np.zeros(max(16, 2 * n), dtype=np.int32), 0, table]
            self._mirror[(group, request)] = rec
        arr, filled, _ = rec
        if n > arr.shape[0]:
            grown = np.zeros(2 * n, dtype=np.int32)
            grown[:filled] = arr[:filled]
            rec[0] = arr = grown
        if n < filled:
            rec[1] = filled = n
        if n > filled:
            arr[filled:n] = [max(p, 0) for p in table[filled:n]]
            rec[1] = n
        return arr[:n]

    def forget(self, request) -> None:
        """Drop what the runner remembers about a request that was released."""
        for gi in self.cache.paged:
            self._mirror.pop((gi, request), None)

    # ---- staging ---------------------------------------------------------------------
    def _stage(self, total: int):
        if self._copied is not None:
            self._copied.synchronize()     # the staging buffer is about to be overwritten
        if len(self._mirror) > 8 * self.cache.max_requests + 64:
            self._mirror = {k: v for k, v in self._mirror.items() if self.cache.has(k[1])}
        if self._pinned is None or self._pinned.numel() < total:
            cap = max(4096, 2 * total)
            self._pinned = torch.empty(cap, dtype=torch.int32).pin_memory() if torch.cuda.is_available() \
                else torch.empty(cap, dtype=torch.int32)
            self._meta = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self._pinned.numpy()

    # ---- the step --------------------------------------------------------------------
    def step(self, entries: list):
        if not entries:
            return None
        cache = self.cache
        seen = set()
        starts, qlens, seqlens, slots_b = [], [], [], []
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request!r} brings no tokens")
            start = cache.num_tokens(e.request)
            cache.ensure(e.request, start + n)     # a no-op when the scheduler has reserved
            starts.append(start)
            qlens.append(n)
            seqlens.append(start + n)
            slots_b.append(cache.state_slot(e.request))
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")
        T, B = sum(qlens), len(entries)
        N = sum(len(e.want) for e in entries)
        groups = cache.paged
        rows = {g: [self._table_row(g, e.request) for e in entries] for g in groups}
        widths = {g: max(1, max(r.shape[0] for r in rows[g])) for g in groups}

        # layout of the one int32 buffer
        layout, off = {}, 0

        def place(name, n):
            nonlocal off
            layout[name] = (off, n)
            off += (n + 3) // 4 * 4        # keep every array 16-byte aligned
        for name, n in (("token_ids", T), ("positions", T), ("token_request", T), ("cu_seqlens", B + 1),
                        ("seq_lens", B), ("logit_rows", N), ("state_slots", B), ("first_portion", B)):
            place(name, n)
        for g in groups:
            place(f"slots{g}", T)
            place(f"table{g}", B * widths[g])
        host = self._stage(off)

        def put(name, values):
            o, n = layout[name]
            host[o:o + n] = values

        ids = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=T)
        if ids.min() < 0 or ids.max() >= self.vocab:
            raise ValueError(f"token id out of range [0, {self.vocab}) in this step")
        put("token_ids", ids)
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(qlens, out=cu[1:])
        put("positions", np.concatenate([np.arange(s, s + n) for s, n in zip(starts, qlens)]))
        put("token_request", np.repeat(np.arange(B), qlens))
        put("cu_seqlens", cu)
        put("seq_lens", seqlens)
        put("logit_rows", [int(cu[b]) + w for b, e in enumerate(entries) for w in e.want])
        put("state_slots", slots_b)
        put("first_portion", [1 if s == 0 else 0 for s in starts])
        ps = cache.page_size
        slots_host = {}
        for g in groups:
            slots = np.concatenate([
                rows[g][b][np.arange(s, s + n) // ps].astype(np.int64) * ps + np.arange(s, s + n) % ps
                for b, (s, n) in enumerate(zip(starts, qlens))])
            put(f"slots{g}", slots)
            slots_host[g] = slots
            o, _ = layout[f"table{g}"]
            tab = host[o:o + B * widths[g]].reshape(B, widths[g])
            tab[:] = 0
            for b, r in enumerate(rows[g]):
                tab[b, :r.shape[0]] = r
        self._meta[:off].copy_(self._pinned[:off], non_blocking=True)
        if self._meta.is_cuda:
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()

        def dev(name):
            o, n = layout[name]
            return self._meta[o:o + n]

        token_request, positions = dev("token_request"), dev("positions")
        cu_dev, seq_dev = dev("cu_seqlens"), dev("seq_lens")
        metas = {}
        for g in groups:
            o, _ = layout[f"table{g}"]
            metas[g] = GroupMeta(block_table=self._meta[o:o + B * widths[g]].view(B, widths[g]),
                                 slots=dev(f"slots{g}"), token_request=token_request, positions=positions,
                                 query_lens=qlens, seq_lens_host=seqlens, cu_seqlens=cu_dev, seq_lens=seq_dev)
        ctx = StepContext(num_tokens=T, num_requests=B, num_logits=N, token_ids=dev("token_ids"),
                          positions=positions, token_request=token_request, cu_seqlens=cu_dev, seq_lens=seq_dev,
                          logit_rows=dev("logit_rows"), state_slots=dev("state_slots"),
                          first_portion=dev("first_portion"), groups=metas, cache=cache,
                          workspace=self.workspace, requests=[e.request for e in entries],
                          query_lens=qlens, starts=starts, slots_host=slots_b)
        logits = self.model.forward(ctx)
        for e, end in zip(entries, seqlens):
            cache.advance(e.request, end)
        self.steps += 1
        return logits
