"""The engine's kernel set: thin, checked wrappers around the sm_100a CUDA library.

`load()` builds `csrc/` on first use, loads the shared library with ctypes and returns the
one `Kernels` object the parts call into.  There is no other implementation: without a
CUDA device of compute capability 10.x, or without a working build, `load()` raises.

Every wrapper takes torch tensors that live on the GPU, checks dtype, shape and layout,
and launches on torch's current stream.  Matrix products in float32 always run this
library's FMA kernel.  In bfloat16 they run this library's tcgen05 kernels where those are
the faster ones (every product of a decode step of up to 32 tokens; the fused SwiGLU product
up to 128 tokens and, on the CTA-pair kernel, from 640 tokens), else cuBLAS through torch
(`torch.mm`), the library the reference's engine uses for them (engine/model.py:194,
F.linear); `gemm_policy` holds the measurements behind the choice.
"""
from __future__ import annotations

import ctypes
import math
import os
import threading

import numpy as np
import torch

from ..csrc import build as _build

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    # name: argtypes (all return int)
    "llm_check_device": [],
    "llm_set_pdl": [_c_int],
    "llm_abi_version": [],
    "llm_embed": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "llm_add_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int,
                        _c_float, _c_int, ctypes.c_longlong, _c_void_p],
    "llm_rope_table": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p],
    "llm_rope_store": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                       _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, ctypes.c_longlong, _c_void_p],
    "llm_silu_mul": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "llm_scale_f32": [_c_void_p, _c_float, ctypes.c_longlong, _c_void_p],
    "llm_sum_parts": [_c_void_p, _c_void_p, _c_int, _c_int, ctypes.c_longlong, _c_void_p],
    "llm_attention_generic": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                              _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "llm_attention_bf16_supported": [_c_int, _c_int, _c_int],
    "llm_attention_prefill_bf16": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "llm_attention_decode_bf16": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                  _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                  _c_float, _c_int, _c_int, _c_void_p],
    "llm_attention_decode_bf16_fused": [_c_void_p, _c_int, ctypes.c_longlong, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                        _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p],
    "llm_attention_decode_tma_supported": [_c_int, _c_int, _c_int, _c_int],
    "llm_attention_decode_bf16_tma": [_c_void_p, _c_int, _c_void_p, ctypes.c_longlong, _c_void_p, _c_int, _c_void_p, _c_int,
                                      _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                                      _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p],
    "llm_attention_decode_bf16_fused_tma": [_c_void_p, _c_int, ctypes.c_longlong, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                            ctypes.c_longlong, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                            _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_float, _c_int, _c_int, _c_void_p],
    "llm_attention_tcgen05_supported": [_c_int, _c_int, _c_int, _c_int],
    "llm_attention_prefill_tcgen05": [_c_void_p, _c_int, _c_int, _c_void_p, ctypes.c_longlong, _c_void_p, _c_int, _c_void_p,
                                      _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                      _c_void_p, _c_void_p, _c_void_p],
    "llm_attention_tcgen05_status": [],
    "llm_gemm_f32": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                     _c_void_p],
    "llm_gemm_bf16_token_tile": [_c_int],
    "llm_gemm_bf16": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                      _c_int, _c_int, _c_int, _c_void_p],
    "llm_gemm_bf16_status": [],
    "llm_gemm_bf16_wait_probe": [_c_int, _c_void_p],
    "llm_gemm_bf16_pair": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                           _c_void_p, _c_void_p],
    "llm_gemm_bf16_pair_scratch": [_c_int],
    "llm_gemm_bf16_pair_status": [],
    "llm_gather_tokens": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p],
    "llm_sample_scratch_floats": [_c_int, _c_int],
    "llm_sample": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "llm_attention_decode_status": [],
}

# The library's health words in the order llm_sample copies them out (csrc/common.cuh): which kernel, and what its codes mean.
HEALTH_WORDS = (
    ("tcgen05 matrix product", "a bounded wait ran out (1 producer, 2 MMA issuer, 3 epilogue)"),
    ("CTA-pair matrix product", "a bounded wait ran out (1 producer, 2 MMA issuer, 3 epilogue, 4 drained accumulator, "
                                "5 other clusters' partial sums)"),
    ("tcgen05 prefill attention", "a bounded wait ran out (1 to 8), or a key's score lay more than 2^100 above all keys of "
                                  "the tiles before it (9: beyond what the one-pass softmax can mend; IITJ_ATTN_ONE_PASS=0 runs two passes "
                                  "everywhere)"),
    ("decode attention", "keys_per_split * max_splits did not cover an item's keys (6), or a bounded wait for keys and "
                         "values ran out (7)"),
)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _check(t, name, dtype=None, dims=None):
    # the usual case in one expression (this runs several times per kernel launch); the messages are made below
    if type(t) is torch.Tensor and t.is_cuda and t.is_contiguous() and (dims is None or t.dim() == dims) and \
            (dtype is None or (t.dtype is dtype if type(dtype) is torch.dtype else t.dtype in dtype)):
        return
    _need(isinstance(t, torch.Tensor), f"{name}: expected a tensor")
    _need(t.is_cuda, f"{name}: tensor is on {t.device}, the kernels run on the GPU only")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list)) else t.dtype == dtype
        _need(ok, f"{name}: dtype {t.dtype} not accepted (want {dtype})")
    if dims is not None:
        _need(t.dim() == dims, f"{name}: expected {dims} dims, got shape {tuple(t.shape)}")
    _need(t.is_contiguous(), f"{name}: tensor must be contiguous")


class PartialSums:
    """The result of a matrix product that was split along k and whose partial sums are still to be added:
    `parts` [splits, tokens, n] float32 (in this library's scratch: valid until the next split product on the
    stream), `out` the tensor the sum belongs in.  `Kernels.add_rmsnorm` and `Kernels.rope_store` take it in
    place of the tensor and add the parts while they read; `sum()` adds them into `out` by a kernel of its own."""

    def __init__(self, kernels, parts, out):
        self.k, self.parts, self.out = kernels, parts, out
        self.shape, self.dtype = out.shape, out.dtype

    @property
    def splits(self) -> int:
        return self.parts.shape[0]

    @property
    def stride(self) -> int:
        return self.parts.shape[1] * self.parts.shape[2]

    def sum(self):
        return self.k.sum_parts(self.parts, self.out)


def materialize(x):
    """The tensor of `x`, which may be a PartialSums."""
    return x.sum() if isinstance(x, PartialSums) else x


class AttentionPlan:
    """How one step's tokens are handed to the tensor-core attention kernels: requests that
    bring one token go to the split-key decode kernel (`items`: their token rows), the rest
    are cut into tiles of 64 queries for the prefill kernel (`tiles`: first token row, rows,
    position of the first row, request).

    It is also the step plan of the attention mixer (parts/base.py, StepPlan): `arrays` are the lists the
    step function copies to the device with its own index arrays, `bind` receives them back as device
    tensors, `graph_key` is what a captured graph freezes of the plan."""

    graph_key = ()
    arrays: dict = {}

    def bind(self, views: dict) -> None:
        self.items = views.get("items")
        self.tiles = views["tiles"].view(-1, 4) if "tiles" in views else None
        self.big_tiles = views["big_tiles"].view(-1, 4) if "big_tiles" in views else None

    TILE = 64
    SPLIT_RULE = os.environ.get("IITJ_DECODE_SPLIT", "auto")    # "equal": always the rule for equal contexts (measurements)
    FORCE_KPS = int(os.environ.get("IITJ_DECODE_KPS", "0"))     # keys per split, whatever the rule says (measurements)

    def __init__(self, query_lens, seq_lens, device, items=None, tiles=None, total_tokens=None):
        self.decode_pos = []
        item_rows, tile_rows, big_rows, row = [], [], [], 0
        if total_tokens is not None and total_tokens == len(query_lens):      # one token each: all decode items
            item_rows, self.decode_pos, query_lens = list(range(total_tokens)), [t - 1 for t in seq_lens], ()
        for b, (n, total) in enumerate(zip(query_lens, seq_lens)):
            if n == 1:
                item_rows.append(row)
                self.decode_pos.append(total - 1)
            else:
                for s in range(0, n, self.TILE):
                    tile_rows.append((row + s, min(self.TILE, n - s), total - n + s, b))
                for s in range(0, n, 2 * self.TILE):        # 128-query tiles of the tcgen05 kernel
                    big_rows.append((row + s, min(2 * self.TILE, n - s), total - n + s, b))
            row += n
        # shortest contexts first: the prefill kernels walk these lists from their ends, so that the tiles with the most
        # keys start first and the short ones fill the gaps at the end of the launch
        big_rows.sort(key=lambda r: r[2] + r[1])
        tile_rows.sort(key=lambda r: r[2] + r[1])
        self.big_rows, self.big_tiles = big_rows, None
        self.n_items, self.n_tiles = len(item_rows), len(tile_rows)
        self.items, self.tiles = items, tiles
        self.context_bound = None     # an upper bound of the contexts that fixes the split choice (captured graphs)
        if self.items is None and item_rows:
            self.items = torch.tensor(item_rows, dtype=torch.int32).to(device)
        if self.tiles is None and tile_rows:
            self.tiles = torch.tensor(tile_rows, dtype=torch.int32).to(device)
        self.item_rows, self.tile_rows = item_rows, tile_rows
        self._splits: dict = {}

    def split(self, kv_heads: int, window: int, sm_count: int, head_dim: int = 128, bound: int | None = None):
        """(keys per split, most splits of any item).

        The decode kernel runs one CTA per (item, key/value head, split of that item's keys); an item with
        fewer keys than `keys per split` has one CTA, a long one several.  `resident` CTAs run at a time (2 per
        SM at head size 128, 4 at 64).  Candidates (the longest context cut into 1 .. 64 parts) are scored in
        units of keys, a CTA costing its keys plus 192:
          * contexts of about equal length (the shortest at least three quarters of the longest): waves of
            `resident` CTAs times the cost of one, which favours cuts that fill whole waves; the best wins;
          * unequal contexts (continuous batching: one 16k-token context beside thirty short ones): the longer
            of the longest CTA times the waves that the CTAs of more than half its length need, and the cost
            of all CTAs together shared out over `resident`; the coarsest cut within 5 % of the best wins.  So
            a long context among short ones is cut into many CTAs instead of keeping one SM busy while the
            others idle.
        `bound` replaces the longest context by an upper bound (captured graphs use one so that the choice
        stays the same while contexts grow); the other contexts are taken as grown by as much."""
        key = (kv_heads, window, head_dim, bound)
        if key not in self._splits:
            spans = []
            for pos in self.decode_pos:
                lo = max(0, pos - window + 1) if window > 0 else 0
                spans.append(pos - (lo // self.TILE) * self.TILE + 1)
            longest = max(spans) if bound is None else max(bound, max(spans))
            resident = sm_count * (2 if head_dim > 64 else 4)
            grown = longest - max(spans)
            equal = 4 * (min(spans) + grown) >= 3 * longest or self.SPLIT_RULE == "equal"
            arr = None if equal else np.asarray(spans, dtype=np.int64) + grown
            keys = 0 if equal else int(arr.sum()) * kv_heads
            pairs = self.n_items * kv_heads
            scored, seen = [], set()
            for n in range(1, 65):
                kps = -(-(-(-longest // n)) // self.TILE) * self.TILE
                if n > 1 and kps < 256:
                    break
                if kps in seen:
                    continue
                seen.add(kps)
                if equal:
                    cost = -(-pairs * -(-longest // kps) // resident) * (kps + 192)
                else:
                    ctas = int((-(-arr // kps)).sum()) * kv_heads
                    long_ctas = int(((arr + kps // 2) // kps).sum()) * kv_heads
                    cost = max(max(1, -(-long_ctas // resident)) * (min(kps, longest) + 192), (keys + 192 * ctas) / resident)
                scored.append((cost, kps))
            least = min(c for c, _ in scored)
            kps = next(k for c, k in scored if c <= (least if equal else 1.05 * least))
            if self.FORCE_KPS:
                kps = self.FORCE_KPS
            self._splits[key] = (kps, max((s - 1) // kps + 1 for s in ([longest] if bound is not None else spans)))
        return self._splits[key]


def attention_plan(meta, device) -> AttentionPlan:
    plan = getattr(meta, "attention_plan", None)
    if plan is None:
        plan = AttentionPlan(meta.query_lens, meta.seq_lens_host, device)
        meta.attention_plan = plan
    return plan


class Kernels:
    """Checked entry points of libllm_kernels.so.  One instance per process (see `load`)."""

    def __init__(self, library_path: str):
        self.library_path = library_path
        self.lib = ctypes.CDLL(library_path)
        self.lib.llm_last_error.restype = ctypes.c_char_p
        for name, args in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes = args
            fn.restype = _c_int
        self.launches = 0  # kernels of this library launched so far (the bench reports it)
        # IITJ_GEMM_BACKEND=cublas|tcgen05 forces one matrix-product path, IITJ_GEMM_SMALL_TOKENS moves the
        # SwiGLU boundary, IITJ_PDL=0 switches programmatic dependent launch off (all for measurements)
        self.gemm_backend = os.environ.get("IITJ_GEMM_BACKEND", "auto")
        self.gemm_small_tokens = int(os.environ.get("IITJ_GEMM_SMALL_TOKENS", "128"))
        self.gemm_plain_tokens = int(os.environ.get("IITJ_GEMM_PLAIN_TOKENS", "128"))   # plain products: tcgen05 up to here
        self.gemm_pair_mode = os.environ.get("IITJ_GEMM_PAIR", "swiglu")   # off | swiglu | all
        self.defer_sums = os.environ.get("IITJ_DEFER_SUMS", "1") == "1"     # k-split sums added by the reading kernel
        self.swiglu_half_tokens = int(os.environ.get("IITJ_SWIGLU_HALF_TOKENS", "64"))  # half-tile SwiGLU product up to here
        self.swiglu_half_smem_kb = int(os.environ.get("IITJ_SWIGLU_HALF_KB", "100"))
        self.fuse_decode = os.environ.get("IITJ_FUSE_DECODE", "1") != "0"   # rope + cache write inside decode attention
        self.decode_tma = os.environ.get("IITJ_DECODE_TMA", "1") != "0"     # decode attention fetches keys and values by TMA
        self.attention_splits = os.environ.get("IITJ_ATTN_SPLITS")         # forces the key splits of prefill attention
        self.attention_tcgen05 = os.environ.get("IITJ_ATTN_TCGEN05", "1") == "1"
        if os.environ.get("IITJ_PDL", "1") == "0":
            self.lib.llm_set_pdl(0)
        self._scratch_bufs: dict = {}
        self._pair_counters: dict = {}
        self._linear_plans: dict = {}    # (tokens, n, k, swiglu) -> (kernel, k-splits, shared memory, half-tile form)
        self.scratch_generation = 0
        self._sm_count = None
        self._device_index = None

    @property
    def sm_count(self) -> int:
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        return self._sm_count

    def _scratch(self, name, floats, device):
        """Grow-only float32 scratch (split-attention partials); contents never outlive a call."""
        buf = self._scratch_bufs.get((name, device))
        if buf is None or buf.numel() < floats:
            buf = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device=device)
            self._scratch_bufs[(name, device)] = buf
            self.scratch_generation += 1
        return buf

    def _scratch_bf16(self, name, elements, device):
        """Grow-only bfloat16 scratch (grown to powers of two, so that token counts that creep up reallocate rarely)."""
        buf = self._scratch_bufs.get((name, device))
        if buf is None or buf.numel() < elements:
            buf = torch.empty(1 << max(elements - 1, 1 << 16).bit_length(), dtype=torch.bfloat16, device=device)
            self._scratch_bufs[(name, device)] = buf
            self.scratch_generation += 1
        return buf[:elements]

    # ---- plumbing --------------------------------------------------------------------
    def _call(self, name, *args):
        rc = getattr(self.lib, name)(*args)
        if rc != 0:
            raise KernelError(f"{name} failed ({rc}): {self.lib.llm_last_error().decode()}")
        self.launches += 1

    def _stream(self):
        """The raw handle of the current CUDA stream (inside a graph capture: the capturing stream)."""
        if self._device_index is None:
            self._device_index = torch.cuda.current_device()
        return torch._C._cuda_getCurrentRawStream(self._device_index)

    def set_pdl(self, on: bool) -> bool:
        """Programmatic dependent launch for all later launches of this library; returns the old setting."""
        return bool(self.lib.llm_set_pdl(1 if on else 0))

    def check_device(self):
        rc = self.lib.llm_check_device()
        if rc != 0:
            raise KernelError(self.lib.llm_last_error().decode())

    def plan_attention(self, shape) -> AttentionPlan:
        """The attention mixer's plan of a step (`shape`: parts.base.StepShape).  For a step that may run from a
        captured graph the split choice of decode attention is fixed by an upper bound of the contexts, in steps of
        512 tokens (the graph is captured anew when the batch outgrows the bound), and a step whose prompt portions
        reach contexts from LONG_PREFILL on is kept apart (its prefill attention launches key splits and a merge)."""
        plan = AttentionPlan(shape.query_lens, shape.seq_lens, shape.device, items=False, tiles=False,
                             total_tokens=shape.num_tokens)
        long_prefill = False
        if shape.graphable:
            if plan.n_items:
                plan.context_bound = (max(plan.decode_pos) + 512) // 512 * 512
            long_prefill = not shape.decode_shaped and any(n > 1 and end >= self.LONG_PREFILL
                                                           for n, end in zip(shape.query_lens, shape.seq_lens))
        plan.graph_key = (plan.context_bound, long_prefill)
        plan.arrays = {}
        if plan.n_items:
            plan.arrays["items"] = plan.item_rows
        if plan.n_tiles:
            plan.arrays["tiles"] = np.asarray(plan.tile_rows, dtype=np.int64).reshape(-1)
            plan.arrays["big_tiles"] = np.asarray(plan.big_rows, dtype=np.int64).reshape(-1)
        return plan

    # ---- row-wise kernels ------------------------------------------------------------
    def embed(self, ids, table, out, scale: float = 1.0):
        """out[t] = scale * table[ids[t]] as float32 (the residual stream)."""
        _check(ids, "embed.ids", torch.int32, 1)
        _check(table, "embed.table", tuple(DTYPE_CODE), 2)
        _check(out, "embed.out", torch.float32, 2)
        _need(out.shape == (ids.shape[0], table.shape[1]), "embed.out: wrong shape")
        self._call("llm_embed", _ptr(ids), _ptr(table), DTYPE_CODE[table.dtype], _ptr(out), ids.shape[0],
                   table.shape[1], table.shape[0], float(scale), self._stream())
        return out

    def add_rmsnorm(self, residual, delta, weight, eps: float, out, rows=None):
        """residual += delta (when given, and rows is None); out = rmsnorm(residual[rows]) * weight."""
        _check(residual, "add_rmsnorm.residual", torch.float32, 2)
        width = residual.shape[1]
        _check(out, "add_rmsnorm.out", tuple(DTYPE_CODE), 2)
        _check(weight, "add_rmsnorm.weight", tuple(DTYPE_CODE), 1)
        _need(weight.shape[0] == width and out.shape[1] == width, "add_rmsnorm: widths differ")
        splits, stride = 0, 0
        if isinstance(delta, PartialSums) and (delta.splits > 8 or delta.stride % 4):
            delta = delta.sum()
        if isinstance(delta, PartialSums):
            _need(tuple(delta.shape) == tuple(residual.shape), "add_rmsnorm.delta: shape differs from residual")
            splits, stride, delta = delta.splits, delta.stride, delta.parts
        elif delta is not None:
            _check(delta, "add_rmsnorm.delta", out.dtype, 2)
            _need(delta.shape == residual.shape, "add_rmsnorm.delta: shape differs from residual")
        if rows is not None:
            _check(rows, "add_rmsnorm.rows", torch.int32, 1)
            _need(out.shape[0] == rows.shape[0], "add_rmsnorm.out: one row per entry of rows")
        else:
            _need(out.shape[0] == residual.shape[0], "add_rmsnorm.out: shape differs from residual")
        self._call("llm_add_rmsnorm", _ptr(residual), _ptr(delta), _ptr(rows), _ptr(weight),
                   DTYPE_CODE[weight.dtype], _ptr(out), DTYPE_CODE[out.dtype], out.shape[0], width, float(eps),
                   splits, stride, self._stream())
        return out

    def rope_tables(self, positions, inv_freq, cos, sin):
        """cos[t, i] = cos(positions[t] * inv_freq[i]) and sin likewise, float32 [tokens, rotary_dim/2]."""
        _check(positions, "rope_tables.positions", torch.int32, 1)
        _check(inv_freq, "rope_tables.inv_freq", torch.float32, 1)
        _check(cos, "rope_tables.cos", torch.float32, 2)
        _check(sin, "rope_tables.sin", torch.float32, 2)
        _need(cos.shape == (positions.shape[0], inv_freq.shape[0]) and sin.shape == cos.shape, "rope_tables: wrong table shape")
        self._call("llm_rope_table", _ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), positions.shape[0],
                   inv_freq.shape[0], self._stream())
        return cos, sin

    def rope_store(self, qkv, positions, inv_freq, slots, cache_layer, heads, kv_heads, head_dim, rotary_dim,
                   tables=None):
        """Rotate q (in place) and k, store k and v of every token in its cache slot.

        cache_layer: [pages, 2, kv_heads, page_size, head_dim]; slots may be None (rotate only).
        tables: (cos, sin) of `rope_tables` for these positions, else the angles are evaluated here.
        `qkv` may be a PartialSums: its parts are added on the way (all dims rotated, head_dim % 8 == 0),
        else summed first.  Returns the tensor that holds the rotated queries."""
        parts = None
        if isinstance(qkv, PartialSums):
            if rotary_dim == head_dim and head_dim % 8 == 0 and qkv.splits <= 8:
                parts, qkv = qkv, qkv.out
            else:
                qkv = qkv.sum()
        _check(qkv, "rope_store.qkv", tuple(DTYPE_CODE), 2)
        _check(positions, "rope_store.positions", torch.int32, 1)
        tokens = qkv.shape[0]
        _need(qkv.shape[1] == (heads + 2 * kv_heads) * head_dim, "rope_store.qkv: width is not (heads+2*kv_heads)*head_dim")
        _need(positions.shape[0] == tokens, "rope_store.positions: one per token")
        if rotary_dim:
            _check(inv_freq, "rope_store.inv_freq", torch.float32, 1)
            _need(inv_freq.shape[0] == rotary_dim // 2, "rope_store.inv_freq: rotary_dim/2 entries")
        page_size = 1
        if slots is not None:
            _check(slots, "rope_store.slots", torch.int32, 1)
            _need(slots.shape[0] == tokens, "rope_store.slots: one per token")
            _check(cache_layer, "rope_store.cache", qkv.dtype, 5)
            _need(cache_layer.shape[1] == 2 and cache_layer.shape[2] == kv_heads and cache_layer.shape[4] == head_dim,
                  f"rope_store.cache: shape {tuple(cache_layer.shape)} does not fit kv_heads/head_dim")
            page_size = cache_layer.shape[3]
        cos = sin = None
        if tables is not None and rotary_dim:
            cos, sin = tables
            _check(cos, "rope_store.cos", torch.float32, 2)
            _check(sin, "rope_store.sin", torch.float32, 2)
            _need(cos.shape == (tokens, rotary_dim // 2) and sin.shape == cos.shape, "rope_store: wrong table shape")
        self._call("llm_rope_store", _ptr(qkv), _ptr(positions), _ptr(inv_freq) if rotary_dim else None, _ptr(cos), _ptr(sin),
                   _ptr(slots), _ptr(cache_layer) if slots is not None else None, DTYPE_CODE[qkv.dtype], tokens,
                   heads, kv_heads, head_dim, rotary_dim, page_size, _ptr(parts.parts) if parts is not None else None,
                   parts.splits if parts is not None else 0, parts.stride if parts is not None else 0, self._stream())
        return qkv

    def silu_mul(self, gu, act):
        _check(gu, "silu_mul.gu", tuple(DTYPE_CODE), 2)
        _check(act, "silu_mul.act", gu.dtype, 2)
        _need(gu.shape[1] == 2 * act.shape[1] and gu.shape[0] == act.shape[0], "silu_mul: shapes do not fit")
        self._call("llm_silu_mul", _ptr(gu), _ptr(act), DTYPE_CODE[gu.dtype], act.shape[0], act.shape[1],
                   self._stream())
        return act

    # ---- attention -------------------------------------------------------------------
    def attention(self, qkv, cache_layer, meta, out, heads, kv_heads, head_dim, window: int = 0,
                  scale: float = 0.0):
        """Causal attention of every token in `qkv` (query heads first in each row) over the
        paged keys and values of its request.  `meta` carries block_table [B, W],
        token_request [T] and positions [T] as int32 device tensors."""
        _check(qkv, "attention.qkv", tuple(DTYPE_CODE), 2)
        _check(cache_layer, "attention.cache", qkv.dtype, 5)
        _check(out, "attention.out", qkv.dtype, 2)
        tokens = qkv.shape[0]
        _need(qkv.shape[1] >= heads * head_dim, "attention.qkv: row too narrow")
        _need(out.shape == (tokens, heads * head_dim), "attention.out: wrong shape")
        _need(cache_layer.shape[1] == 2 and cache_layer.shape[2] == kv_heads and cache_layer.shape[4] == head_dim,
              f"attention.cache: shape {tuple(cache_layer.shape)} does not fit kv_heads/head_dim")
        _check(meta.block_table, "attention.block_table", torch.int32, 2)
        _check(meta.token_request, "attention.token_request", torch.int32, 1)
        _check(meta.positions, "attention.positions", torch.int32, 1)
        _need(meta.token_request.shape[0] == tokens and meta.positions.shape[0] == tokens,
              "attention: one token_request and one position per token")
        if not scale:
            scale = 1.0 / math.sqrt(head_dim)
        page_size = cache_layer.shape[3]
        if qkv.dtype == torch.bfloat16 and self.lib.llm_attention_bf16_supported(heads, kv_heads, head_dim):
            plan = attention_plan(meta, qkv.device)
            if plan.n_tiles and self.attention_tcgen05 and \
                    cache_layer.shape[0] * 2 * kv_heads * page_size < (1 << 31) and \
                    self.lib.llm_attention_tcgen05_supported(heads, kv_heads, head_dim, page_size):     # (TMA coordinates are 32-bit)
                if plan.big_tiles is None:
                    plan.big_tiles = torch.tensor(plan.big_rows, dtype=torch.int32).to(qkv.device)
                splits = self.prefill_key_splits(plan.big_rows, heads, kv_heads, int(window))
                part_o = part_ml = None
                if splits > 1:
                    n = len(plan.big_rows) * heads * splits * 128
                    part_o = self._scratch("attn.tc_part_o", n * head_dim, qkv.device)
                    part_ml = self._scratch("attn.tc_part_ml", n * 2, qkv.device)
                self._call("llm_attention_prefill_tcgen05", _ptr(qkv), qkv.shape[1], tokens, _ptr(cache_layer),
                           cache_layer.shape[0], _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.big_tiles),
                           len(plan.big_rows), _ptr(out), out.shape[1], heads, kv_heads, head_dim, page_size, int(window),
                           float(scale), splits, _ptr(part_o), _ptr(part_ml), self._stream())
                if splits > 1:
                    self.launches += 1
            elif plan.n_tiles:
                self._call("llm_attention_prefill_bf16", _ptr(qkv), qkv.shape[1], _ptr(cache_layer),
                           _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.tiles), plan.n_tiles, _ptr(out),
                           out.shape[1], heads, kv_heads, head_dim, page_size, int(window), float(scale), self._stream())
            if plan.n_items:
                kps, splits = plan.split(kv_heads, int(window), self.sm_count, head_dim, getattr(plan, 'context_bound', None))
                part_o = part_ml = None
                if splits > 1:
                    part_o = self._scratch("attn.part_o", plan.n_items * heads * splits * head_dim, qkv.device)
                    part_ml = self._scratch("attn.part_ml", plan.n_items * heads * splits * 2, qkv.device)
                if self._decode_by_tma(cache_layer, heads, kv_heads, head_dim):
                    self._call("llm_attention_decode_bf16_tma", _ptr(qkv), qkv.shape[1], _ptr(cache_layer), cache_layer.shape[0],
                               _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.items), plan.n_items,
                               _ptr(meta.token_request), _ptr(meta.positions), _ptr(part_o), _ptr(part_ml), _ptr(out),
                               out.shape[1], heads, kv_heads, head_dim, page_size, int(window), float(scale), kps, splits,
                               self._stream())
                else:
                    self._call("llm_attention_decode_bf16", _ptr(qkv), qkv.shape[1], _ptr(cache_layer),
                               _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.items), plan.n_items,
                               _ptr(meta.token_request), _ptr(meta.positions), _ptr(part_o), _ptr(part_ml), _ptr(out),
                               out.shape[1], heads, kv_heads, head_dim, page_size, int(window), float(scale), kps, splits,
                               self._stream())
                if splits > 1:
                    self.launches += 1      # the merge kernel
            return out
        self._call("llm_attention_generic", _ptr(qkv), qkv.shape[1], _ptr(cache_layer), _ptr(meta.block_table),
                   meta.block_table.shape[1], _ptr(meta.token_request), _ptr(meta.positions), _ptr(out),
                   out.shape[1], DTYPE_CODE[qkv.dtype], tokens, heads, kv_heads, head_dim, page_size,
                   int(window), float(scale), self._stream())
        return out

    def _decode_by_tma(self, cache_layer, heads, kv_heads, head_dim) -> bool:
        """True if decode attention fetches this cache layer's keys and values by TMA: a page size of 8 to 64 tokens, and
        a layer whose rows (pages x 2 x kv_heads x page_size) fit TMA's 32-bit coordinates; else the copying kernel runs."""
        pages, page_size = cache_layer.shape[0], cache_layer.shape[3]
        return bool(self.decode_tma and pages * 2 * kv_heads * page_size < (1 << 31) and
                    self.lib.llm_attention_decode_tma_supported(heads, kv_heads, head_dim, page_size))

    def can_fuse_decode(self, qkv, meta, cache_layer, heads, kv_heads, head_dim) -> bool:
        """True if `attention_decode_fused` takes this step: every token is a single decoded token, the qkv
        product was left as at most eight partial sums, bfloat16 cache, a shape of the tensor-core kernel."""
        if not (self.fuse_decode and isinstance(qkv, PartialSums) and 1 <= qkv.splits <= 8 and qkv.stride % 4 == 0):
            return False
        if cache_layer is None or cache_layer.dtype != torch.bfloat16 or qkv.out.dtype != torch.bfloat16:
            return False
        if not self.lib.llm_attention_bf16_supported(heads, kv_heads, head_dim):
            return False
        plan = attention_plan(meta, cache_layer.device)
        return plan.n_tiles == 0 and plan.n_items == qkv.out.shape[0]

    def attention_decode_fused(self, qkv, tables, slots, cache_layer, meta, out, heads, kv_heads, head_dim,
                               window: int = 0, scale: float = 0.0):
        """Decode attention straight from the qkv product's partial sums (`can_fuse_decode` holds): adds the
        parts, rotates queries and keys with `tables` (cos, sin of `rope_tables`; every dim rotated), stores each
        token's key and value at `slots`, attends over the paged cache.  One kernel (and the merge of key
        splits) in place of rope_store + attention."""
        cos, sin = tables
        tokens = qkv.out.shape[0]
        _check(qkv.parts, "attention_decode_fused.parts", torch.float32, 3)
        _check(cos, "attention_decode_fused.cos", torch.float32, 2)
        _check(sin, "attention_decode_fused.sin", torch.float32, 2)
        _check(slots, "attention_decode_fused.slots", torch.int32, 1)
        _check(cache_layer, "attention_decode_fused.cache", torch.bfloat16, 5)
        _check(out, "attention_decode_fused.out", torch.bfloat16, 2)
        _need(qkv.out.shape[1] == (heads + 2 * kv_heads) * head_dim, "attention_decode_fused: qkv width is not (heads+2*kv_heads)*head_dim")
        _need(cos.shape == (tokens, head_dim // 2) and sin.shape == cos.shape, "attention_decode_fused: tables must be [tokens, head_dim/2]")
        _need(slots.shape[0] == tokens and out.shape == (tokens, heads * head_dim), "attention_decode_fused: one slot and one output row per token")
        _need(cache_layer.shape[1] == 2 and cache_layer.shape[2] == kv_heads and cache_layer.shape[4] == head_dim,
              f"attention_decode_fused.cache: shape {tuple(cache_layer.shape)} does not fit kv_heads/head_dim")
        _need(meta.token_request.shape[0] == tokens and meta.positions.shape[0] == tokens,
              "attention_decode_fused: one token_request and one position per token")
        if not scale:
            scale = 1.0 / math.sqrt(head_dim)
        plan = attention_plan(meta, out.device)
        _need(plan.n_tiles == 0 and plan.n_items == tokens, "attention_decode_fused: every token must be a single decoded token")
        kps, splits = plan.split(kv_heads, int(window), self.sm_count, head_dim, getattr(plan, 'context_bound', None))
        part_o = part_ml = None
        if splits > 1:
            part_o = self._scratch("attn.part_o", plan.n_items * heads * splits * head_dim, out.device)
            part_ml = self._scratch("attn.part_ml", plan.n_items * heads * splits * 2, out.device)
        if self._decode_by_tma(cache_layer, heads, kv_heads, head_dim):
            self._call("llm_attention_decode_bf16_fused_tma", _ptr(qkv.parts), qkv.splits, qkv.stride, _ptr(cos), _ptr(sin),
                       _ptr(slots), _ptr(cache_layer), cache_layer.shape[0], _ptr(meta.block_table), meta.block_table.shape[1],
                       _ptr(plan.items), plan.n_items, _ptr(meta.token_request), _ptr(meta.positions), _ptr(part_o),
                       _ptr(part_ml), _ptr(out), out.shape[1], heads, kv_heads, head_dim, cache_layer.shape[3], int(window),
                       float(scale), kps, splits, self._stream())
        else:
            self._call("llm_attention_decode_bf16_fused", _ptr(qkv.parts), qkv.splits, qkv.stride, _ptr(cos), _ptr(sin), _ptr(slots),
                       _ptr(cache_layer), _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.items), plan.n_items,
                       _ptr(meta.token_request), _ptr(meta.positions), _ptr(part_o), _ptr(part_ml), _ptr(out), out.shape[1],
                       heads, kv_heads, head_dim, cache_layer.shape[3], int(window), float(scale), kps, splits, self._stream())
        if splits > 1:
            self.launches += 1      # the merge kernel
        return out

    # ---- matrix products -------------------------------------------------------------
    def prefill_key_splits(self, big_rows, heads, kv_heads, window) -> int:
        """CTAs along the keys of each 128-query tile of the tcgen05 prefill attention.  The kernel is at its best
        with two heads per CTA and about 1.7 CTAs per SM; a short portion of a prompt against a long context has
        too few query tiles for that, so its keys are shared out.  This is the number of CTAs the launch provides
        per tile and head; the kernel uses as many of them as leave each about 16 key tiles of 128, by the tile's
        own context (a captured graph thus follows a prompt as it grows).
        Measured at 32 heads / 8 key-value heads: 512 queries over 16384 keys 260 -> 209 us with 4 splits, over
        32768 keys 510 -> 352 us; 128 queries over 16384 keys 254 -> 86 us."""
        if self.attention_splits is not None:
            return max(1, min(16, int(self.attention_splits)))
        longest = max(min(pos0 + rows, window + rows) if window > 0 else pos0 + rows for _, rows, pos0, _ in big_rows)
        if longest < self.LONG_PREFILL:               # no tile would use a second split: no merge kernel either
            return 1
        group = heads // kv_heads
        pair_ctas = len(big_rows) * kv_heads * ((group + 1) // 2)
        splits = max(1, min(16, round(1.7 * self.sm_count / pair_ctas)))
        if pair_ctas * splits < self.sm_count:        # too few even so: the kernel then runs one head per CTA
            splits = max(1, min(16, self.sm_count // (len(big_rows) * heads)))
        return splits

    # Context from which a query tile's keys may be shared out over two CTAs (24 key tiles of 128).  A step's
    # captured graph freezes whether its prefill attention launches splits at all, so the step function keeps
    # shorter and longer contexts apart in its graph keys.
    LONG_PREFILL = 3072

    def linear(self, x, weight, out, swiglu: bool = False, defer: bool = False):
        """out = x . weight^T; with swiglu, weight holds gate rows then up rows and
        out = silu(x . gate^T) * (x . up^T).  With `defer` the result may come back as a PartialSums (the product
        was split along k and the caller's next kernel adds the parts); else `out`."""
        _check(x, "linear.x", tuple(DTYPE_CODE), 2)
        _check(weight, "linear.weight", x.dtype, 2)
        _check(out, "linear.out", (x.dtype, torch.float32), 2)
        n = weight.shape[0] // 2 if swiglu else weight.shape[0]
        _need(x.shape[1] == weight.shape[1], f"linear: x has {x.shape[1]} columns, weight {weight.shape[1]}")
        _need(out.shape == (x.shape[0], n), f"linear.out: shape {tuple(out.shape)}, want {(x.shape[0], n)}")
        if x.shape[0] == 0:
            return out
        if x.dtype == torch.float32:
            self._call("llm_gemm_f32", _ptr(x), _ptr(weight), _ptr(out), x.shape[0], n, x.shape[1], x.shape[1],
                       weight.shape[1], n, 1 if swiglu else 0, self._stream())
            return out
        # bfloat16: this library's tcgen05 kernel where it is the faster one, else cuBLAS through torch
        tokens, k = x.shape
        # which kernel, and how it is cut, depends on the shape alone: decided once per shape
        pkey = (tokens, n, k, swiglu)
        plan = self._linear_plans.get(pkey)
        if plan is None:
            policy = self.gemm_policy(tokens, n, k, swiglu)
            if policy == "tcgen05":
                if swiglu and tokens <= self.swiglu_half_tokens and n % 64 == 0:
                    # decode batches: 64 gate + 64 up rows per CTA, twice the CTAs (two per SM), no k-split and no kernel
                    # after it.  Against the whole tile (128 + 128 rows, one CTA per SM, 112 CTAs at the 8B shape) a decode
                    # step at 4096-token contexts: batch 16 / 32 at the 8B shape 4.61 -> 4.57 / 5.98 -> 5.93 ms, batch 32 / 64
                    # at the 3B shape 4.43 -> 4.31 / 7.54 -> 7.42 ms, at the 1B shape 1.97 -> 1.88 / 3.11 -> 3.03 ms; level at
                    # batch 64 of the 8B shape and at batch 128, where the whole tile stays
                    plan = ("tcgen05", 1, self.swiglu_half_smem_kb, True)
                else:
                    plan = ("tcgen05",) + tuple(self.gemm_plan(tokens, n, k, swiglu)) + (False,)
            else:
                plan = (policy, 1, 0, False)
            if len(self._linear_plans) > 8192:
                self._linear_plans.clear()
            self._linear_plans[pkey] = plan
        policy, splits, smem_kb, half = plan
        if policy == "tcgen05":
            if half:
                return self.gemm_tcgen05(x, weight, out, True, 1, smem_kb, half=True)
            return self.gemm_tcgen05(x, weight, out, swiglu, splits, smem_kb, defer=defer and not swiglu and self.defer_sums)
        if policy == "pair":
            return self.gemm_pair(x, weight, out, swiglu)
        if swiglu:
            # the [tokens, 2 * inner] intermediate lives in this library's grow-only scratch: a step allocates nothing
            gu = self._scratch_bf16("gemm.gate_up", tokens * weight.shape[0], x.device).view(tokens, weight.shape[0])
            torch.mm(x, weight.t(), out=gu)
            return self.silu_mul(gu, out)
        if out.dtype == torch.float32:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, weight.t(), out=out)
        return out

    def gemm_tcgen05(self, x, weight, out, swiglu: bool = False, splits: int = 1, smem_kb: int = 0, defer: bool = False,
                     half: bool = False):
        """out = x . weight^T on this library's tcgen05 kernel (bfloat16 in, bfloat16 or float32 out).  With `defer`
        and more than one split the partial sums are returned as a PartialSums instead of being added here.
        `half`: the SwiGLU product of at most 128 tokens with 64 gate and 64 up rows per CTA (unsplit, n % 64 == 0)."""
        _check(x, "gemm.x", torch.bfloat16, 2)
        _check(weight, "gemm.weight", torch.bfloat16, 2)
        _check(out, "gemm.out", (torch.bfloat16, torch.float32), 2)
        tokens, k = x.shape
        n = weight.shape[0] // 2 if swiglu else weight.shape[0]
        _need(weight.shape[1] == k and out.shape == (tokens, n), "gemm: shapes do not fit")
        splits = max(1, min(int(splits), -(-k // 64)))
        scratch = None
        if splits > 1:
            scratch = self._scratch("gemm.partials", splits * tokens * weight.shape[0], x.device)
        defer = bool(defer and splits > 1 and not swiglu)
        self._call("llm_gemm_bf16", _ptr(x), _ptr(weight), _ptr(out), 1 if out.dtype == torch.float32 else 0, tokens,
                   n, k, out.shape[1], 1 if swiglu else 0, splits, _ptr(scratch), int(smem_kb), 1 if defer else 0,
                   1 if half else 0, self._stream())
        if defer:
            return PartialSums(self, scratch[:splits * tokens * n].view(splits, tokens, n), out)
        if splits > 1:
            self.launches += 1
        return out

    def sum_parts(self, parts, out):
        """out = the sum over the first dimension of `parts` [splits, tokens, n] float32, added in split order."""
        _check(parts, "sum_parts.parts", torch.float32, 3)
        _check(out, "sum_parts.out", tuple(DTYPE_CODE), 2)
        _need(tuple(parts.shape[1:]) == tuple(out.shape), "sum_parts: shapes do not fit")
        self._call("llm_sum_parts", _ptr(parts), _ptr(out), DTYPE_CODE[out.dtype], parts.shape[0], out.numel(), self._stream())
        return out

    def scale_(self, x, scale: float):
        """x *= scale, float32, in place."""
        _check(x, "scale_.x", torch.float32)
        self._call("llm_scale_f32", _ptr(x), float(scale), x.numel(), self._stream())
        return x

    def gemm_pair(self, x, weight, out, swiglu: bool = False, tail_split: bool = True):
        """out = x . weight^T on this library's persistent CTA-pair tcgen05 kernel (many tokens).  With
        `tail_split` the tiles of the last, partly filled round are cut along k over all clusters."""
        _check(x, "gemm.x", torch.bfloat16, 2)
        _check(weight, "gemm.weight", torch.bfloat16, 2)
        _check(out, "gemm.out", (torch.bfloat16, torch.float32), 2)
        tokens, k = x.shape
        n = weight.shape[0] // 2 if swiglu else weight.shape[0]
        _need(weight.shape[1] == k and out.shape == (tokens, n), "gemm: shapes do not fit")
        partials = counters = None
        if tail_split:
            partials = self._scratch("gemm.pair.partials", self.lib.llm_gemm_bf16_pair_scratch(0), x.device)
            counters = self._pair_counters.get(x.device)
            if counters is None:      # zeroed once; every launch leaves them zero again
                counters = torch.zeros(self.lib.llm_gemm_bf16_pair_scratch(1), dtype=torch.int32, device=x.device)
                self._pair_counters[x.device] = counters
        self._call("llm_gemm_bf16_pair", _ptr(x), _ptr(weight), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                   tokens, n, k, out.shape[1], 1 if swiglu else 0, _ptr(partials), _ptr(counters), self._stream())
        return out

    # Which kernel multiplies: "tcgen05" (this library) or "cublas".  `gemm_backend` may force one.
    def gemm_policy(self, tokens, n, k, swiglu) -> str:
        """"tcgen05" (one CTA per tile, weights on the 128-row side), "pair" (persistent CTA pairs, tokens on
        the 256-row side) or "cublas".  Measured on B200 at the 8B shapes, in CUDA graphs with cold weights:
        up to 32 tokens the tcgen05 product with two or three CTAs per SM and up to eight k-splits matches
        or beats cuBLAS for every shape of the model (and its weight prefetch overlaps the kernel before
        it); from there to 128 tokens it is 5-17 % behind by itself, but its k-split sums are added by the
        kernels that read them and the decode attention takes them with the rotation fused in, so the whole
        decode step is 3-5 % faster with it (batch 48 / 64 / 128 at 8192-token contexts: 12.4 -> 11.8, 15.3 ->
        14.9, 27.7 -> 26.9 ms); beyond 128 tokens cuBLAS wins (batch 192: 14.6 against 15.2 ms).  The fused
        SwiGLU form holds up to 128 tokens.  From about 640 tokens the pair kernel's fused
        SwiGLU product beats cuBLAS plus a separate activation kernel (2048 tokens: 330 against 365 us).  Its
        plain products stay about 7 % behind cuBLAS, which halves its operand traffic with multicast loads
        that this library does not use, so those stay on cuBLAS (IITJ_GEMM_PAIR=all moves them over)."""
        if k % 8:
            return "cublas"
        if self.gemm_backend != "auto":
            return self.gemm_backend
        if tokens <= (self.gemm_small_tokens if swiglu else min(self.gemm_plain_tokens, self.gemm_small_tokens)):
            return "tcgen05"
        if tokens >= 640 and (self.gemm_pair_mode == "all" or (swiglu and self.gemm_pair_mode == "swiglu")):
            return "pair"
        return "cublas"

    def gemm_plan(self, tokens, n, k, swiglu) -> tuple:
        """(k-splits, shared memory per CTA in KiB) for the tcgen05 product.

        Products with many feature tiles (the LM head) run unsplit with three CTAs per SM.  Products with
        few tiles are split along k until about two CTAs per SM are in flight (at most eight splits, at
        least four k-blocks each).  The SwiGLU product beyond the half-tile form's token count (see linear) runs
        unsplit with the whole shared memory as its ring."""
        tile = self.lib.llm_gemm_bf16_token_tile(tokens)
        tiles = -(-n // 128) * -(-tokens // tile)
        k_blocks = -(-k // 64)
        if tokens > 256 or n % 4:
            return 1, 0
        if tiles >= 2 * self.sm_count:
            return 1, 66
        if swiglu and tokens > 8:
            return 1, 0
        splits = max(1, min(8, round(2 * self.sm_count / tiles), k_blocks // 4))
        return splits, 100

    def gemm_splits(self, tokens, n, k, swiglu) -> int:
        return self.gemm_plan(tokens, n, k, swiglu)[0]

    def gemm_status(self) -> int:
        """0, or a code if a tcgen05 GEMM gave up waiting on one of its barriers since the last call."""
        return self.lib.llm_gemm_bf16_status()

    def wait_probe(self, polls: int = 2000) -> None:
        """Launches a kernel whose only act is a bounded wait that runs out after `polls` polls (an mbarrier nobody
        arrives on; nothing else is in flight); it leaves code 7 in the tcgen05 product's status word.  For tests of
        what the host makes of a kernel that gave up."""
        self._call("llm_gemm_bf16_wait_probe", int(polls), self._stream())

    def gemm_pair_status(self) -> int:
        """0, or a code if the CTA-pair GEMM gave up waiting on one of its barriers since the last call."""
        return self.lib.llm_gemm_bf16_pair_status()

    def attention_status(self) -> int:
        """0, or a code if the tcgen05 attention kernel gave up waiting on a barrier since the last call."""
        return self.lib.llm_attention_tcgen05_status()

    def decode_status(self) -> int:
        """0, or a code if a decode attention call since the last read was given too few splits for an item's keys."""
        return self.lib.llm_attention_decode_status()

    HEALTH_WORDS = len(HEALTH_WORDS)

    def check_health(self, codes=None) -> None:
        """Raises KernelError if a kernel of this library reported that it gave up (a bounded wait that ran out) or
        that a contract was broken since the last check; what such a kernel wrote cannot be used.  `codes`: the
        words as `sample(..., health=...)` copied them out; None reads them from the device now (which waits for
        the work in flight).  On a failure the device words are cleared and the CTA-pair product's tile counters,
        which a CTA that gave up may have left non-zero, are zeroed again, so the library can be used afterwards."""
        if codes is None:
            codes = [self.gemm_status(), self.gemm_pair_status(), self.attention_status(), self.decode_status()]
        codes = [int(c) for c in codes]
        if not any(codes):
            return
        self.gemm_status(), self.gemm_pair_status(), self.attention_status(), self.decode_status()   # read = clear
        for counters in self._pair_counters.values():
            counters.zero_()
        bad = [f"{name}: code {c >> 16} in block/item {c & 0xffff} ({meaning})"
               for c, (name, meaning) in zip(codes, HEALTH_WORDS) if c]
        raise KernelError("a kernel gave up, its output is not valid: " + "; ".join(bad))

    def gather_tokens(self, dst, src, rows):
        """dst[i] = src[rows[i]] where rows[i] >= 0 (int32 device tensors): the previous step's sampled ids
        become this step's input tokens without a trip to the host."""
        _check(dst, "gather_tokens.dst", torch.int32, 1)
        _check(src, "gather_tokens.src", torch.int32, 1)
        _check(rows, "gather_tokens.rows", torch.int32, 1)
        _need(rows.shape[0] == dst.shape[0], "gather_tokens: one source row per destination")
        self._call("llm_gather_tokens", _ptr(dst), _ptr(src), _ptr(rows), dst.shape[0], self._stream())

    # ---- sampling --------------------------------------------------------------------
    def sample(self, logits, temperature, keys, out, health=None):
        """out[r] = argmax of row r (temperature[r] <= 0) or a draw from softmax(row / T).  `health`: an int32 tensor
        of HEALTH_WORDS entries that receives the library's status words (see `check_health`)."""
        _check(logits, "sample.logits", torch.float32, 2)
        _check(out, "sample.out", torch.int32, 1)
        rows = logits.shape[0]
        _need(out.shape[0] == rows, "sample.out: one per row")
        if temperature is not None:
            _check(temperature, "sample.temperature", torch.float32, 1)
            _check(keys, "sample.keys", torch.int64, 1)
            _need(temperature.shape[0] == rows and keys.shape[0] == rows, "sample: one temperature and key per row")
        if health is not None:
            _check(health, "sample.health", torch.int32, 1)
            _need(health.shape[0] >= self.HEALTH_WORDS, "sample.health: too short")
        need = self.lib.llm_sample_scratch_floats(rows, logits.shape[1])
        scratch = self._scratch("sample.part", need, logits.device) if need else None
        self._call("llm_sample", _ptr(logits), logits.shape[1], _ptr(temperature), _ptr(keys), _ptr(out), rows,
                   logits.shape[1], _ptr(scratch), _ptr(health), self._stream())
        return out


_lock = threading.Lock()
_instance = None


def load() -> Kernels:
    """The process-wide kernel set; builds and loads the library on first call."""
    global _instance
    with _lock:
        if _instance is None:
            if not torch.cuda.is_available():
                raise KernelError("no CUDA device is visible: this engine runs on the GPU only "
                                  "(there is no CPU path)")
            k = Kernels(_build.library_path())
            k.check_device()
            _instance = k
        return _instance
