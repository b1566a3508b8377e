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

Parts may need index arrays of their own (an attention kernel's tile lists): the step function
asks every part that implements `prepare_step` (parts/base.py) once per step, places the arrays
it returns in the same buffer, hands them back as device views, and folds the part's `graph_key`
into the key under which the step's CUDA graph is kept.  It knows no part by name.
"""
from __future__ import annotations

import gc
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheError
from ..parts.base import Part, StepShape
from .context import GroupMeta, StepContext, Workspace


_no_plan = Part.prepare_step       # the base class's "nothing to plan"


@dataclass
class StepEntry:
    request: object
    tokens: list
    want: list = field(default_factory=list)   # indices into `tokens`
    source_rows: list | None = None            # per token: row of the previous step's sampled ids that holds it
    #                                            (the host does not know it yet), or -1 for a token given here


class ModelRunner:
    def __init__(self, model, cache, device="cuda", cuda_graphs: bool = False):
        self.model, self.cache, self.device = model, cache, device
        self.use_graphs = bool(cuda_graphs) and str(device).startswith("cuda") and \
            bool(getattr(model, "graph_safe", False))
        self._graphs: dict = {}      # key -> captured decode step
        self._graph_seen: dict = {}  # key -> eager runs so far
        self.graph_replays = 0
        self.graph_captures = 0
        self.padded_steps = 0
        # A step shape is captured into a graph once it has been seen this often: a capture costs about as much as
        # ten eager steps, so shapes that come and go (a batch that shrinks every few steps) are not worth one.
        self.graph_after = 3
        self.vocab = model.spec.vocab
        self.workspace = Workspace(device)
        self._pinned = None          # int32 staging buffer (host, pinned)
        self._meta = None            # int32 device buffer the step's index arrays live in
        self._copied = None          # event: the last host-to-device copy of the staging buffer is done
        self._capture_stream = None  # side stream that graph captures are recorded on
        self.steps = 0
        self.copied_bytes = 0
        self._preparer_list = None

    def _preparers(self) -> list:
        """(prepare_key, part) of every part of the model that plans per-step arrays, one per key."""
        if self._preparer_list is None:
            found = {}
            for part in getattr(self.model, "all_parts", lambda: [])():
                if getattr(type(part), "prepare_step", _no_plan) is not _no_plan:
                    found.setdefault(getattr(part, "prepare_key", None) or id(part), part)
            self._preparer_list = list(found.items())
        return self._preparer_list

    # ---- staging ---------------------------------------------------------------------
    def _stage(self, total: int):
        if self._copied is not None:
            self._copied.synchronize()     # the staging buffer is about to be overwritten
        if self._pinned is None or self._pinned.numel() < total:
            cap = max(4096, 2 * total)
            self._pinned = torch.empty(cap, dtype=torch.int32).pin_memory() if torch.cuda.is_available() \
                else torch.empty(cap, dtype=torch.int32)
            self._meta = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self._pinned.numpy()

    # ---- captured decode steps --------------------------------------------------------
    def _generation(self):
        k = getattr(self.model, "k", None)
        return (self.workspace.generation, getattr(k, "scratch_generation", 0), self._meta.data_ptr())

    def _forward_graphed(self, key, ctx, eager_runs: int = 1):
        """Runs a step whose shape is `key`: eagerly the first `eager_runs` times that shape is seen
        (which also brings every scratch buffer to size), captured into a CUDA graph the next time,
        replayed from then on.  The index arrays were copied to their fixed places before."""
        rec = self._graphs.get(key)
        if rec is not None and rec["generation"] == self._generation():
            rec["graph"].replay()
            self.graph_replays += 1
            k = getattr(self.model, "k", None)
            if k is not None:
                k.launches += rec["launches"]
            return rec["logits"]
        if self._graph_seen.get(key, 0) < eager_runs:
            if len(self._graph_seen) > 4096:
                self._graph_seen.clear()
            self._graph_seen[key] = self._graph_seen.get(key, 0) + 1
            return self.model.forward(ctx)
        if len(self._graphs) >= 64:
            self._graphs.pop(next(iter(self._graphs)))
        k = getattr(self.model, "k", None)
        before = k.launches if k is not None else 0
        generation = self._generation()
        self.graph_captures += 1
        graph = torch.cuda.CUDAGraph()
        # The garbage collector must not run inside the capture: collecting an older engine there would
        # destroy its graphs, which CUDA forbids while a capture is open and which voids the capture.
        # The capture is opened by hand rather than with torch.cuda.graph(), which first waits for the whole
        # device and empties the allocator's cache: a step may be in flight, and the step's buffers exist already.
        gc_was_on = gc.isenabled()
        gc.disable()
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream()
        self._capture_stream.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(self._capture_stream):
                graph.capture_begin(capture_error_mode="thread_local")
                try:
                    logits = self.model.forward(ctx)
                finally:
                    graph.capture_end()
        finally:
            if gc_was_on:
                gc.enable()
        launches = (k.launches - before) if k is not None else 0
        if generation != self._generation():     # a buffer grew while capturing: do not keep the graph
            self._graph_seen[key] = 0
            return self.model.forward(ctx)
        self._graphs[key] = {"graph": graph, "logits": logits, "generation": generation, "launches": launches}
        graph.replay()
        self.graph_replays += 1
        return logits

    @staticmethod
    def _padded_batch(b: int) -> int:
        """The batch size a decode step of `b` requests runs at: itself up to 8, then the next multiple of 8
        (to 64), of 16 (to 128), of 32."""
        if b <= 8:
            return b
        step = 8 if b <= 64 else 16 if b <= 128 else 32
        return -(-b // step) * step

    # ---- the step --------------------------------------------------------------------
    def step(self, entries: list, prev_ids=None):
        """`prev_ids`: the previous step's sampled ids on the device, for entries with `source_rows`."""
        if not entries:
            return None
        cache = self.cache
        stored, room, slot_of = cache.stored, cache.room, cache.slot_of
        starts, qlens, slots_b = [], [], []
        N = 0
        for e in entries:
            r, n = e.request, len(e.tokens)
            if n == 0:
                raise ValueError(f"request {r!r} brings no tokens")
            start = stored.get(r)
            if start is None:
                raise CacheError(f"request {r!r} is not admitted to the cache (admit it before its first step)")
            if start + n > room[r]:
                cache.ensure(r, start + n)         # (the scheduler has reserved already: this is the replay's path)
            starts.append(start)
            qlens.append(n)
            slots_b.append(slot_of[r])
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {r!r}: wanted place {w} is outside its {n} tokens")
            N += len(e.want)
        B = len(entries)
        if len(set(slots_b)) != B:
            twice = next(e.request for i, e in enumerate(entries) if slots_b[i] in slots_b[:i])
            raise ValueError(f"request {twice!r} appears twice in one step")
        T = sum(qlens)
        groups = cache.paged
        # A decode step (one token and one wanted row per request) is padded to the next batch size of a short
        # ladder, so that batches which shrink by a request every few steps still meet captured graphs.  A padding
        # row is a one-token request at position 0 whose block table and state slot are the cache's padding page
        # and slot; its logits row is cut off below.
        pad = 0
        if self.use_graphs and T == B and N == B:
            pad = self._padded_batch(B) - B
        if pad:
            self.padded_steps += 1
            starts += [0] * pad
            qlens += [1] * pad
            slots_b += [cache.pad_slot] * pad
            T, B, N = T + pad, B + pad, N + pad
        decode_shaped = T == B and N == B
        q, st = np.asarray(qlens, dtype=np.int64), np.asarray(starts, dtype=np.int64)
        slot_rows = np.asarray(slots_b, dtype=np.int64)
        seqlens = (st + q).tolist()
        # the block tables come from the cache manager's matrix (one row per state slot) in one gather per group
        widths = {g: max(1, int(cache.groups[g].lengths[slot_rows].max())) for g in groups}
        # A step whose shape (tokens per request, wanted rows, table width) has been seen before can be
        # replayed from a captured graph if the index arrays keep their places, so the block tables are
        # padded to a power of two of pages.  Decode steps repeat at once; prompt portions of the same
        # length (a chunked prefill under a token budget) repeat too.
        graphable = self.use_graphs
        if graphable:
            widths = {g: max(16, 1 << (w - 1).bit_length()) for g, w in widths.items()}
        # the parts' own index arrays and what a graph freezes of them
        shape = StepShape(query_lens=qlens, seq_lens=seqlens, num_tokens=T, decode_shaped=decode_shaped,
                          graphable=graphable, device=self.device)
        prepared = {}
        for key, part in self._preparers():
            plan = part.prepare_step(shape)
            if plan is not None:
                prepared[key] = plan

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
        fed = prev_ids is not None and any(e.source_rows is not None for e in entries)
        if fed:
            place("token_src", T)
        for key, plan in prepared.items():
            for name, values in plan.arrays.items():
                place(f"{key}.{name}", len(values))
        old_meta = self._meta
        host = self._stage(off)
        if self._meta is not old_meta:
            self._graphs.clear()           # the index arrays moved: captured graphs point at the old buffer

        def put(name, values):
            o, n = layout[name]
            host[o:o + n] = values

        ids = np.zeros(T, dtype=np.int64)
        ids[:T - pad] = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=T - pad)
        if fed:
            src = np.full(T, -1, dtype=np.int64)
            if decode_shaped:
                src[:T - pad] = [e.source_rows[0] if e.source_rows is not None else -1 for e in entries]
            else:
                src[:T - pad] = [r for e in entries
                                 for r in (e.source_rows if e.source_rows is not None else [-1] * len(e.tokens))]
            put("token_src", src)
            ids = np.where(src >= 0, 0, ids)          # placeholders: the device fills them in
        if ids.min() < 0 or ids.max() >= self.vocab:
            raise ValueError(f"token id out of range [0, {self.vocab}) in this step")
        put("token_ids", ids)
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(q, out=cu[1:])
        if T == B:
            token_request, positions = np.arange(B), st
        else:
            token_request = np.repeat(np.arange(B), q)
            positions = np.arange(T) - np.repeat(cu[:-1] - st, q)
        put("positions", positions)
        put("token_request", token_request)
        put("cu_seqlens", cu)
        put("seq_lens", seqlens)
        if decode_shaped:
            put("logit_rows", cu[:-1])
        else:
            first = cu.tolist()
            put("logit_rows", [first[b] + w for b, e in enumerate(entries) for w in e.want])
        put("state_slots", slot_rows)
        put("first_portion", st == 0)
        for key, plan in prepared.items():
            for name, values in plan.arrays.items():
                put(f"{key}.{name}", values)
        ps = cache.page_size
        page_of, offset_in = positions // ps, positions % ps
        for g in groups:
            matrix = cache.groups[g].matrix
            o, _ = layout[f"table{g}"]
            tab = host[o:o + B * widths[g]].reshape(B, widths[g])
            cols = min(widths[g], matrix.shape[1])
            tab[:, :cols] = matrix[slot_rows, :cols]
            tab[:, cols:] = 0
            put(f"slots{g}", tab[token_request, page_of].astype(np.int64) * ps + offset_in)
        self._meta[:off].copy_(self._pinned[:off], non_blocking=True)
        self.copied_bytes = 4 * off            # what this step sent to the device (benchmarks report it)
        if self._meta.is_cuda:
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()

        def dev(name):
            o, n = layout[name]
            return self._meta[o:o + n]

        if fed:
            self.model.k.gather_tokens(dev("token_ids"), prev_ids, dev("token_src"))
        for key, plan in prepared.items():
            plan.bind({name: dev(f"{key}.{name}") for name in plan.arrays})
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
                          workspace=self.workspace, requests=[e.request for e in entries] + [None] * pad,
                          query_lens=qlens, starts=starts, slots_host=slots_b, prepared=prepared)
        if graphable:
            form = ("decode", B) if decode_shaped else (tuple(qlens), tuple(len(e.want) for e in entries))
            key = (form, tuple(sorted(widths.items())), fed, tuple((k, p.graph_key) for k, p in prepared.items()))
            logits = self._forward_graphed(key, ctx, eager_runs=self.graph_after if decode_shaped else max(4, self.graph_after))
        else:
            logits = self.model.forward(ctx)
        cache.advance_all([e.request for e in entries], seqlens)
        self.steps += 1
        if pad and logits is not None:
            logits = logits[:N - pad]
        return logits
