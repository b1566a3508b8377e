"""The allocation-free decode attention entry point, called through its exported C symbol.

`llm_attention_decode_bf16_static` serves callers that reach this library from outside
PyTorch (a C serving shell, another language's FFI) and cannot, or must not, allocate
device memory where they call: its split partials live in an array built into the
library.  The test calls the symbol with ctypes exactly as such a caller would (raw
pointers, nothing allocated in between), twice in a row on different inputs so that the
second call runs over what the first left in the shared array, and compares each result
with the ordinary entry point, which is given scratch by its caller, and with the plain
restatement of paged attention in tests/torch_kernels.py.

This file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes
import math
from types import SimpleNamespace

import pytest
import torch

import torch_kernels as R

pytestmark = pytest.mark.gpu

TOL = 1.6e-2      # the bfloat16 tolerance of tests/test_kernels_gpu.py


def _case(seed, lens, heads, kv_heads, head_dim, page):
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // page) for n in lens]
    total_pages = sum(need) + 2
    perm = iter(torch.randperm(total_pages, generator=g).tolist())
    table = torch.zeros(len(lens), max(need), dtype=torch.int32)
    for b, n in enumerate(need):
        for j in range(n):
            table[b, j] = next(perm)
    gd = torch.Generator(device="cuda").manual_seed(seed)
    cache = torch.randn((total_pages, 2, kv_heads, page, head_dim), generator=gd, device="cuda").to(torch.bfloat16)
    q = torch.randn((len(lens), (heads + 2 * kv_heads) * head_dim), generator=gd, device="cuda").to(torch.bfloat16)
    meta = SimpleNamespace(block_table=table.cuda(), token_request=torch.arange(len(lens), dtype=torch.int32).cuda(),
                           positions=torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda(),
                           query_lens=[1] * len(lens), seq_lens_host=list(lens))
    return q, cache, meta


def test_static_scratch_entry_point_matches_the_ordinary_one_twice():
    from iitj_llm_coopt_b200 import kernels
    K = kernels.load()
    fn = K.lib.llm_attention_decode_bf16_static          # the exported C symbol
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, ci, vp, vp, ci, vp, ci, vp, vp, vp, ci, ci, ci, ci, ci, ci, ctypes.c_float, ci, ci, vp]
    fn.restype = ci
    heads, kv_heads, head_dim, page = 8, 2, 128, 16
    kps = 256
    for seed, lens in ((1, [700, 300, 1000, 257, 64]), (2, [1500, 90, 513])):
        q, cache, meta = _case(seed, lens, heads, kv_heads, head_dim, page)
        want = torch.empty(len(lens), heads * head_dim, device="cuda", dtype=torch.bfloat16)
        K.attention(q, cache, meta, want, heads, kv_heads, head_dim)          # ordinary path, caller-owned scratch
        items = torch.arange(len(lens), dtype=torch.int32, device="cuda")
        out = torch.zeros_like(want)
        splits = max((n - 1) // kps + 1 for n in lens)
        torch.cuda.synchronize()
        rc = fn(q.data_ptr(), q.shape[1], cache.data_ptr(), meta.block_table.data_ptr(), meta.block_table.shape[1],
                items.data_ptr(), len(lens), meta.token_request.data_ptr(), meta.positions.data_ptr(), out.data_ptr(),
                out.shape[1], heads, kv_heads, head_dim, page, 0, 1.0 / math.sqrt(head_dim), kps, splits,
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0, K.lib.llm_last_error().decode()
        torch.cuda.synchronize()
        err = (out.float() - want.float()).abs().max().item()
        assert err <= TOL * want.float().abs().max().item(), err
        plain = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads, head_dim)
        err = (out.float() - plain).abs().max().item()
        assert err <= TOL * plain.abs().max().item(), err
    assert K.decode_status() == 0


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from iitj_llm_coopt_b200 import kernels
    K = kernels.load()
    fn = K.lib.llm_attention_decode_bf16_static
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, ci, vp, vp, ci, vp, ci, vp, vp, vp, ci, ci, ci, ci, ci, ci, ctypes.c_float, ci, ci, vp]
    fn.restype = ci
    dummy = torch.zeros(16, device="cuda", dtype=torch.int32)
    # 4096 items x 32 heads x 16 splits x 130 floats is far beyond the 2M floats of the array;
    # the size check comes before anything is read or launched
    rc = fn(dummy.data_ptr(), 1, dummy.data_ptr(), dummy.data_ptr(), 1, dummy.data_ptr(), 4096, dummy.data_ptr(),
            dummy.data_ptr(), dummy.data_ptr(), 1, 32, 8, 128, 16, 0, 0.1, 256, 16, None)
    assert rc < 0
    msg = K.lib.llm_last_error().decode()
    assert "scratch" in msg and "2097152" in msg


def test_too_few_splits_are_reported_and_stay_inside_their_partials():
    """A caller that passes max_splits one too small for its longest item breaks the entry point's contract.  The
    kernels cut that item down to max_splits: nothing outside the item's own partials is read or written (the other
    items' results stay right, and so does the memory after the output), the item's last keys are left out (its
    result is the attention over the keys that were covered), and the status word says so."""
    from iitj_llm_coopt_b200 import kernels
    K = kernels.load()
    fn = K.lib.llm_attention_decode_bf16_static
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, ci, vp, vp, ci, vp, ci, vp, vp, vp, ci, ci, ci, ci, ci, ci, ctypes.c_float, ci, ci, vp]
    fn.restype = ci
    heads, kv_heads, head_dim, page, kps = 8, 2, 128, 16, 256
    lens = [500, 1000, 300]                              # the second needs four splits of 256 keys; it gets three
    q, cache, meta = _case(3, lens, heads, kv_heads, head_dim, page)
    items = torch.arange(len(lens), dtype=torch.int32, device="cuda")
    guard = 4096
    buf = torch.full((len(lens) * heads * head_dim + guard,), 7.0, device="cuda", dtype=torch.bfloat16)
    out = buf[:len(lens) * heads * head_dim].view(len(lens), heads * head_dim)
    K.decode_status()                                    # start from a clear word
    rc = fn(q.data_ptr(), q.shape[1], cache.data_ptr(), meta.block_table.data_ptr(), meta.block_table.shape[1],
            items.data_ptr(), len(lens), meta.token_request.data_ptr(), meta.positions.data_ptr(), out.data_ptr(),
            out.shape[1], heads, kv_heads, head_dim, page, 0, 1.0 / math.sqrt(head_dim), kps, 3,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, K.lib.llm_last_error().decode()
    torch.cuda.synchronize()
    code = K.decode_status()
    assert code >> 16 == 6 and code & 0xffff == 1, hex(code)
    assert K.decode_status() == 0                        # reading cleared it
    assert bool((buf[len(lens) * heads * head_dim:] == 7.0).all())
    plain = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads, head_dim)
    for b in (0, 2):
        assert (out[b].float() - plain[b]).abs().max().item() <= TOL * plain.abs().max().item()
    # the cut item: attention over its first 3 * 256 keys, by the plain restatement with the position moved back
    short = meta.positions.clone()
    short[1] = 3 * kps - 1
    covered = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, short, heads, kv_heads, head_dim)
    assert (out[1].float() - covered[1]).abs().max().item() <= TOL * covered.abs().max().item()
