"""Each CUDA kernel alone against its plain-torch restatement (tests/torch_kernels.py), at
sizes other than the engine's test models: widths and vocabularies that are no power of
two, head sizes in steps of 16, odd numbers of heads and groups, several page sizes."""
import math
from types import SimpleNamespace

import pytest
import torch

import torch_kernels as R

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}   # relative to the largest reference magnitude


@pytest.fixture(scope="module")
def K():
    from iitj_llm_coopt_b200 import kernels
    return kernels.load()


def close(got, want, dtype, scale=1.0):
    err = (got.float() - want.float()).abs().max().item()
    ref = max(want.float().abs().max().item(), 1e-20)
    assert err <= TOL[dtype] * scale * ref, (err, ref)


def rnd(shape, dtype, seed, std=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * std).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,width,tokens", [(320, 96, 7), (1000, 200, 33)])
def test_embed(K, dtype, vocab, width, tokens):
    table = rnd((vocab, width), dtype, 1)
    ids = torch.randint(0, vocab, (tokens,), device="cuda", dtype=torch.int32)
    ids[0], ids[-1] = 0, vocab - 1
    out = torch.empty(tokens, width, device="cuda")
    K.embed(ids, table, out, 1.5)
    assert torch.equal(out, R.ref_embed(ids, table, 1.5))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("rows,width,eps", [(5, 96, 1e-6), (19, 200, 1e-5), (3, 4104, 1e-5), (2, 13000, 1e-5)])
def test_add_rmsnorm(K, dtype, wdtype, rows, width, eps):
    res = rnd((rows, width), torch.float32, 2)
    delta = rnd((rows, width), dtype, 3)
    w = (1 + 0.1 * rnd((width,), torch.float32, 4)).to(wdtype)
    # plain norm, no delta
    out = torch.empty(rows, width, device="cuda", dtype=dtype)
    before = res.clone()
    K.add_rmsnorm(res, None, w, eps, out)
    assert torch.equal(res, before)
    close(out, R.ref_add_rmsnorm(before, None, w, eps)[1], dtype)
    # residual += delta, then norm
    K.add_rmsnorm(res, delta, w, eps, out)
    v, y = R.ref_add_rmsnorm(before, delta, w, eps)
    close(res, v, torch.float32)
    close(out, y, dtype)
    # gathered rows: the residual is left alone
    idx = torch.tensor([rows - 1, 0, rows - 1], device="cuda", dtype=torch.int32)
    out2 = torch.empty(3, width, device="cuda", dtype=dtype)
    keep = res.clone()
    K.add_rmsnorm(res, delta, w, eps, out2, rows=idx)
    assert torch.equal(res, keep)
    close(out2, R.ref_add_rmsnorm(keep, delta, w, eps, rows=idx)[1], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary,page", [(3, 1, 32, 32, 8), (5, 5, 48, 48, 16), (6, 2, 80, 40, 4),
                                                                (4, 2, 128, 128, 64), (2, 1, 16, 0, 16)])
def test_rope_store(K, dtype, heads, kv_heads, head_dim, rotary, page):
    tokens, pages = 23, 9
    qkv = rnd((tokens, (heads + 2 * kv_heads) * head_dim), dtype, 5)
    positions = torch.randint(0, 100000, (tokens,), device="cuda", dtype=torch.int32)
    positions[0] = 0
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, rotary, 2).float() / max(rotary, 1)))).cuda() if rotary else None
    perm = torch.randperm(pages * page, device="cuda")[:tokens].to(torch.int32)
    perm[3] = -1                                   # "do not store" for one token
    cache = torch.full((pages, 2, kv_heads, page, head_dim), 7.0, device="cuda", dtype=dtype)
    want_cache = cache.clone()
    want = R.ref_rope(qkv, positions, inv_freq, heads, kv_heads, head_dim, rotary)
    R.ref_store(want_cache, want.to(dtype), perm, heads, kv_heads, head_dim)
    got = qkv.clone()
    K.rope_store(got, positions, inv_freq, perm, cache, heads, kv_heads, head_dim, rotary)
    q = heads * head_dim
    close(got[:, :q], want[:, :q], dtype)
    close(cache, want_cache, dtype)
    assert torch.equal(cache == 7.0, want_cache == 7.0)          # nothing else was touched
    # with the step's table of cosines and sines
    if rotary:
        cos = torch.empty(tokens, rotary // 2, device="cuda")
        sin = torch.empty_like(cos)
        K.rope_tables(positions, inv_freq, cos, sin)
        got3, cache3 = qkv.clone(), torch.full_like(cache, 7.0)
        K.rope_store(got3, positions, inv_freq, perm, cache3, heads, kv_heads, head_dim, rotary, tables=(cos, sin))
        assert torch.equal(got3, got) and torch.equal(cache3, cache)
    # rotate only (no slots): the cache is not needed
    got2 = qkv.clone()
    K.rope_store(got2, positions, inv_freq, None, None, heads, kv_heads, head_dim, rotary)
    close(got2[:, :q], want[:, :q], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(K, dtype):
    gu = rnd((11, 2 * 176), dtype, 6, 3.0)
    act = torch.empty(11, 176, device="cuda", dtype=dtype)
    K.silu_mul(gu, act)
    close(act, R.ref_silu_mul(gu), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 320, 96), (7, 130, 176), (65, 64, 64), (130, 200, 264), (3, 1000, 4104)])
def test_linear(K, dtype, m, n, k):
    x, w = rnd((m, k), dtype, 7), rnd((n, k), dtype, 8, 0.05)
    out = torch.empty(m, n, device="cuda", dtype=dtype)
    K.linear(x, w, out)
    close(out, R.ref_linear(x, w), dtype)
    out32 = torch.empty(m, n, device="cuda", dtype=torch.float32)
    K.linear(x, w, out32)
    close(out32, R.ref_linear(x, w), torch.float32 if dtype == torch.float32 else dtype, 0.1 if dtype == torch.bfloat16 else 1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 176, 64), (9, 344, 96), (70, 100, 200)])
def test_linear_swiglu(K, dtype, m, n, k):
    x, w = rnd((m, k), dtype, 9), rnd((2 * n, k), dtype, 10, 0.2)
    out = torch.empty(m, n, device="cuda", dtype=dtype)
    K.linear(x, w, out, swiglu=True)
    close(out, R.ref_linear(x, w, swiglu=True), dtype)


def test_linear_row_does_not_depend_on_batch(K):
    """float32: a row's product is the same alone and among 100 others, bit for bit."""
    x, w = rnd((101, 264), torch.float32, 11), rnd((200, 264), torch.float32, 12)
    full = torch.empty(101, 200, device="cuda")
    one = torch.empty(1, 200, device="cuda")
    K.linear(x, w, full)
    K.linear(x[77:78].contiguous(), w, one)
    assert torch.equal(full[77:78], one)


def _paged_case(dtype, heads, kv_heads, head_dim, page, lens, qlens, seed, pages_extra=3):
    """Random paged cache for requests with total lengths `lens`, the last qlens[b] tokens being queries."""
    B = len(lens)
    need = [-(-n // page) for n in lens]
    total_pages = sum(need) + pages_extra
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total_pages, generator=g).tolist()
    width = max(need)
    table = torch.zeros(B, width, dtype=torch.int32)
    it = iter(perm)
    for b in range(B):
        for j in range(need[b]):
            table[b, j] = next(it)
    cache = rnd((total_pages, 2, kv_heads, page, head_dim), dtype, seed + 1)
    T = sum(qlens)
    q = rnd((T, (heads + 2 * kv_heads) * head_dim), dtype, seed + 2)
    token_request = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(qlens)])
    positions = torch.cat([torch.arange(L - n, L, dtype=torch.int32) for L, n in zip(lens, qlens)])
    meta = SimpleNamespace(block_table=table.cuda(), token_request=token_request.cuda(), positions=positions.cuda(),
                           query_lens=list(qlens), seq_lens_host=list(lens))
    return q, cache, meta


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,page,window", [
    (3, 1, 32, 8, 0), (4, 2, 16, 16, 0), (6, 2, 64, 16, 0), (4, 1, 128, 16, 0), (5, 5, 48, 4, 0),
    (2, 1, 80, 32, 0), (8, 2, 256, 16, 0), (4, 2, 64, 16, 20), (3, 1, 32, 8, 7)])
def test_attention_mixed_batch(K, dtype, heads, kv_heads, head_dim, page, window):
    lens, qlens = [70, 33, 150, 1, 17], [70, 1, 13, 1, 2]          # whole prompt, decode, portion, first token, two tokens
    q, cache, meta = _paged_case(dtype, heads, kv_heads, head_dim, page, lens, qlens, 20)
    out = torch.empty(q.shape[0], heads * head_dim, device="cuda", dtype=dtype)
    K.attention(q, cache, meta, out, heads, kv_heads, head_dim, window=window)
    want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads,
                                 head_dim, window)
    close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,page", [(64, 16), (128, 16), (32, 8)])
@pytest.mark.parametrize("far", [0, 15, 16, 17, 255, 256, 700, 1022])
def test_attention_finds_a_far_key(K, dtype, head_dim, page, far):
    """One key among a thousand is made to stand out; the output must be that key's value.
    Positions are chosen on and beside page edges and tile edges."""
    heads, kv_heads, L = 4, 2, 1023
    q, cache, meta = _paged_case(dtype, heads, kv_heads, head_dim, page, [L], [1], 30 + far)
    cache.mul_(0.1)
    pg, off = int(meta.block_table[0, far // page]), far % page
    marker = rnd((kv_heads, head_dim), torch.float32, 99)
    for h in range(heads):
        hk = h // (heads // kv_heads)
        qv = q[0, h * head_dim:(h + 1) * head_dim].float()
        cache[pg, 0, hk, off] = (qv / qv.norm() * 60.0 / (qv.norm() / math.sqrt(head_dim))).to(dtype) \
            if h % (heads // kv_heads) == 0 else cache[pg, 0, hk, off]
    cache[pg, 1, :, off] = marker.to(dtype)
    out = torch.empty(1, heads * head_dim, device="cuda", dtype=dtype)
    K.attention(q, cache, meta, out, heads, kv_heads, head_dim)
    want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads, head_dim)
    close(out, want, dtype)
    first = out[0, :head_dim].float()                      # head 0 looks straight at the far key
    assert (first - marker[0].to(dtype).float()).abs().max() < 0.05 * marker.abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(K, dtype):
    """A key just outside the window must not be seen, the one just inside must."""
    heads, kv_heads, head_dim, page, window, L = 2, 1, 64, 16, 37, 200
    q, cache, meta = _paged_case(dtype, heads, kv_heads, head_dim, page, [L], [1], 41)
    cache.mul_(0.1)
    inside, outside = L - window, L - window - 1
    qv = q[0, :head_dim].float()
    big = (qv / qv.norm() * 60.0 / (qv.norm() / math.sqrt(head_dim))).to(dtype)
    for pos, val in ((inside, 1.0), (outside, -1.0)):
        pg, off = int(meta.block_table[0, pos // page]), pos % page
        cache[pg, 0, 0, off] = big
        cache[pg, 1, 0, off] = val
    out = torch.empty(1, heads * head_dim, device="cuda", dtype=dtype)
    K.attention(q, cache, meta, out, heads, kv_heads, head_dim, window=window)
    want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads,
                                 head_dim, window)
    close(out, want, dtype)
    assert out[0, :head_dim].float().mean() > 0.9


def test_attention_refuses_odd_head_size(K):
    from iitj_llm_coopt_b200.kernels import KernelError
    q, cache, meta = _paged_case(torch.float32, 2, 1, 24, 16, [5], [5], 50)
    out = torch.empty(5, 48, device="cuda")
    with pytest.raises(KernelError):
        K.attention(q, cache, meta, out, 2, 1, 24)


@pytest.mark.parametrize("vocab", [320, 1000, 128256])
def test_sample_greedy_and_ties(K, vocab):
    logits = rnd((6, vocab), torch.float32, 60)
    logits[2, 5] = logits[2, vocab - 3] = 50.0                # a tie: the lowest index wins
    logits[3, vocab - 1] = 60.0
    out = torch.empty(6, device="cuda", dtype=torch.int32)
    K.sample(logits, None, None, out)
    assert out.tolist() == logits.argmax(-1).tolist()
    assert out[2].item() == 5 and out[3].item() == vocab - 1


def test_sample_temperature_matches_reference_stream(K):
    from iitj_llm_coopt_b200.sampling import row_key
    vocab, rows = 1000, 64
    logits = rnd((rows, vocab), torch.float32, 61, 2.0)
    temps = torch.tensor([0.0 if r % 4 == 0 else 0.5 + 0.01 * r for r in range(rows)])
    keys = [row_key(7, r, 3 * r) for r in range(rows)]
    keys_t = torch.tensor([k - (1 << 64) if k >= (1 << 63) else k for k in keys], dtype=torch.int64)
    out = torch.empty(rows, device="cuda", dtype=torch.int32)
    K.sample(logits, temps.cuda(), keys_t.cuda(), out)
    want, perturbed = R.ref_sample(logits.cpu(), temps, keys)
    top2 = perturbed.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 1e-3                  # skip near-ties of the perturbed rows
    assert clear.sum() > rows // 2
    assert torch.equal(out.cpu()[clear], want[clear])
    # the same key gives the same token whatever else is in the batch
    out1 = torch.empty(1, device="cuda", dtype=torch.int32)
    K.sample(logits[5:6].contiguous(), temps[5:6].cuda(), keys_t[5:6].cuda(), out1)
    assert out1.item() == out[5].item()


def test_sample_temperature_follows_softmax(K):
    """Frequencies of 20000 draws from a 5-token distribution against softmax(logits / T)."""
    from iitj_llm_coopt_b200.sampling import row_key
    logits = torch.tensor([[1.0, 2.0, 0.0, 3.0, -1.0]]).repeat(20000, 1).cuda()
    T = 0.8
    keys = [row_key(1, 2, i) for i in range(20000)]
    keys_t = torch.tensor([k - (1 << 64) if k >= (1 << 63) else k for k in keys], dtype=torch.int64).cuda()
    out = torch.empty(20000, device="cuda", dtype=torch.int32)
    K.sample(logits, torch.full((20000,), T).cuda(), keys_t, out)
    freq = torch.bincount(out.long().cpu(), minlength=5).float() / 20000
    want = torch.softmax(logits[0].cpu() / T, -1)
    assert (freq - want).abs().max() < 0.015, (freq, want)


def _poison_unwritten_slots(cache, meta, lens, page):
    """NaN in every slot after a request's last token (the rest of its last page) and in the pages no request
    holds: nothing of them may reach a result."""
    used = set()
    for b, n in enumerate(lens):
        for j in range(-(-n // page)):
            used.add(int(meta.block_table[b, j]))
        if n % page:
            cache[int(meta.block_table[b, (n - 1) // page]), :, :, n % page:, :] = float("nan")
    for pg in range(cache.shape[0]):
        if pg not in used and pg != 0:                  # (page 0 pads the block table's rows)
            cache[pg] = float("nan")


@pytest.mark.parametrize("heads,kv_heads,head_dim,page,window", [
    (8, 2, 128, 16, 0), (32, 8, 128, 16, 0), (16, 1, 64, 16, 0), (6, 2, 64, 8, 0), (4, 4, 128, 32, 0),
    (8, 2, 128, 16, 300), (3, 1, 64, 4, 0), (2, 1, 128, 64, 0), (5, 1, 64, 64, 130), (12, 4, 128, 8, 0)])
def test_attention_bf16_decode_splits(K, decode_loads, heads, kv_heads, head_dim, page, window):
    """Only single-token requests, contexts long enough to be cut into several splits; what lies in the cache after
    a request's last token is NaN."""
    lens = [700, 300, 1000, 257, 64, 65, 1, 1500]
    q, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lens, [1] * len(lens), 70)
    _poison_unwritten_slots(cache, meta, lens, page)
    out = torch.empty(q.shape[0], heads * head_dim, device="cuda", dtype=torch.bfloat16)
    K.attention(q, cache, meta, out, heads, kv_heads, head_dim, window=window)
    want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads,
                                 head_dim, window)
    close(out, want, torch.bfloat16)
    assert K.decode_status() == 0


@pytest.mark.parametrize("heads,kv_heads,head_dim,page,window", [
    (8, 2, 128, 16, 0), (4, 1, 64, 16, 0), (6, 2, 64, 8, 0), (2, 2, 128, 64, 0), (4, 2, 128, 16, 100), (4, 2, 64, 16, 64)])
def test_attention_bf16_prefill_tiles(K, heads, kv_heads, head_dim, page, window):
    """Portions longer than one 64-query tile, starting at positions that are no multiple of 64."""
    lens, qlens = [700, 130, 391, 64], [200, 130, 65, 64]
    q, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lens, qlens, 80)
    out = torch.empty(q.shape[0], heads * head_dim, device="cuda", dtype=torch.bfloat16)
    K.attention(q, cache, meta, out, heads, kv_heads, head_dim, window=window)
    want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads,
                                 head_dim, window)
    close(out, want, torch.bfloat16)


@pytest.mark.parametrize("head_dim,context", [(128, 9000), (64, 5000), (128, 4500), (64, 20000)])
def test_attention_bf16_one_long_request_has_many_splits(K, decode_loads, head_dim, context):
    """One decoded token alone: its keys are cut into more splits than the merge kernel keeps in registers (17 to 31,
    32 and more), and one key that stands out lies in the last but one."""
    from iitj_llm_coopt_b200.kernels import AttentionPlan
    heads, kv_heads, page = 8, 2, 16
    q, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, [context], [1], 95)
    plan = AttentionPlan(meta.query_lens, meta.seq_lens_host, "cuda", total_tokens=1)
    meta.attention_plan = plan
    kps, splits = plan.split(kv_heads, 0, K.sm_count, head_dim, None)
    assert splits > 16, (kps, splits)
    far = (splits - 2) * kps + 5
    direction = rnd((head_dim,), torch.float32, 96)
    direction = direction / direction.norm()
    pg, off = int(meta.block_table[0, far // page]), far % page
    cache[pg, 0, :, off] = (direction * 30.0).to(torch.bfloat16)
    cache[pg, 1, :, off] = 2.0
    q[0, :heads * head_dim] = (direction * 12.0).repeat(heads).to(torch.bfloat16)
    out = torch.empty(1, heads * head_dim, device="cuda", dtype=torch.bfloat16)
    K.attention(q, cache, meta, out, heads, kv_heads, head_dim)
    want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads, head_dim)
    close(out, want, torch.bfloat16)
    assert (out.float() - 2.0).abs().max().item() < 0.1
    assert K.decode_status() == 0


def test_attention_bf16_same_result_in_any_batch(K, decode_loads):
    """A decoded token's output is bitwise the same alone and beside other requests."""
    heads, kv_heads, head_dim, page = 8, 2, 128, 16
    lens, qlens = [500, 130, 77], [1, 40, 1]
    q, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lens, qlens, 90)
    out = torch.empty(q.shape[0], heads * head_dim, device="cuda", dtype=torch.bfloat16)
    K.attention(q, cache, meta, out, heads, kv_heads, head_dim)
    solo = SimpleNamespace(block_table=meta.block_table[2:3].contiguous(), token_request=torch.zeros(1, dtype=torch.int32, device="cuda"),
                           positions=meta.positions[41:42].contiguous(), query_lens=[1], seq_lens_host=[77])
    out1 = torch.empty(1, heads * head_dim, device="cuda", dtype=torch.bfloat16)
    K.attention(q[41:42].contiguous(), cache, solo, out1, heads, kv_heads, head_dim)
    assert torch.equal(out1[0], out[41])


@pytest.mark.parametrize("heads,kv_heads,page,window,splits", [(8, 2, 16, 0, 3), (3, 1, 16, 0, 2), (4, 4, 32, 0, 5),
                                                               (4, 2, 16, 700, 4), (2, 1, 8, 0, 16)])
@pytest.mark.parametrize("head_dim", [128, 64])
def test_attention_tcgen05_key_splits(K, heads, kv_heads, page, window, splits, head_dim):
    """The keys of a query tile shared out over several CTAs whose partial results a merge kernel adds: short
    portions against long contexts, more splits than some tiles have key tiles, a window that leaves early splits
    without a visible key for late rows."""
    lens, qlens = [3000, 1500, 200, 2100], [200, 130, 200, 1]
    q, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lens, qlens, 140)
    want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads, head_dim, window)
    old = K.attention_splits
    try:
        for forced in (splits, None):
            K.attention_splits = forced
            out = torch.zeros(q.shape[0], heads * head_dim, device="cuda", dtype=torch.bfloat16)
            K.attention(q, cache, meta, out, heads, kv_heads, head_dim, window=window)
            close(out, want, torch.bfloat16)
    finally:
        K.attention_splits = old
    assert K.attention_status() == 0


# ---- k-split partial sums added by the kernel that reads the result ------------------------
@pytest.mark.parametrize("rows,width,splits", [(9, 264, 3), (1, 96, 2), (40, 4096, 8), (5, 100, 4)])
def test_add_rmsnorm_partial_sums(K, rows, width, splits):
    from iitj_llm_coopt_b200.kernels import PartialSums
    res = rnd((rows, width), torch.float32, 130)
    parts = rnd((splits, rows, width), torch.float32, 131, 0.3)
    w = (1 + 0.1 * rnd((width,), torch.float32, 132)).to(torch.bfloat16)
    delta = PartialSums(K, parts, torch.empty(rows, width, device="cuda", dtype=torch.bfloat16))
    out = torch.empty(rows, width, device="cuda", dtype=torch.bfloat16)
    before = res.clone()
    K.add_rmsnorm(res, delta, w, 1e-5, out)
    v, y = R.ref_add_rmsnorm(before, parts.sum(0), w, 1e-5)
    close(res, v, torch.float32)
    close(out, y, torch.bfloat16)
    idx = torch.tensor([rows - 1, 0], device="cuda", dtype=torch.int32)
    out2 = torch.empty(2, width, device="cuda", dtype=torch.bfloat16)
    keep = res.clone()
    K.add_rmsnorm(res, delta, w, 1e-5, out2, rows=idx)
    assert torch.equal(res, keep)
    close(out2, R.ref_add_rmsnorm(keep, parts.sum(0), w, 1e-5, rows=idx)[1], torch.bfloat16)
    close(delta.sum(), parts.sum(0), torch.bfloat16)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page,splits", [(4, 2, 32, 8, 3), (3, 1, 128, 16, 2), (8, 8, 64, 16, 5)])
def test_rope_store_partial_sums(K, heads, kv_heads, head_dim, page, splits):
    from iitj_llm_coopt_b200.kernels import PartialSums
    tokens, pages = 11, 6
    width = (heads + 2 * kv_heads) * head_dim
    parts = rnd((splits, tokens, width), torch.float32, 133, 0.5)
    positions = torch.randint(0, 100000, (tokens,), device="cuda", dtype=torch.int32)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))).cuda()
    slots = torch.randperm(pages * page, device="cuda")[:tokens].to(torch.int32)
    slots[2] = -1
    cache = torch.full((pages, 2, kv_heads, page, head_dim), 7.0, device="cuda", dtype=torch.bfloat16)
    want_cache = cache.clone()
    want = R.ref_rope(parts.sum(0), positions, inv_freq, heads, kv_heads, head_dim, head_dim)
    R.ref_store(want_cache, want.to(torch.bfloat16), slots, heads, kv_heads, head_dim)
    qkv = PartialSums(K, parts, torch.zeros(tokens, width, device="cuda", dtype=torch.bfloat16))
    got = K.rope_store(qkv, positions, inv_freq, slots, cache, heads, kv_heads, head_dim, head_dim)
    q = heads * head_dim
    close(got[:, :q], want[:, :q], torch.bfloat16)
    close(cache, want_cache, torch.bfloat16)
    assert torch.equal(cache == 7.0, want_cache == 7.0)
    # a rotation that covers only part of the head: the parts are added first, then the usual kernel runs
    cache2 = torch.full_like(cache, 7.0)
    half_freq = (1.0 / (500000.0 ** (torch.arange(0, head_dim // 2, 2).float() / (head_dim // 2)))).cuda()
    got2 = K.rope_store(PartialSums(K, parts, torch.zeros(tokens, width, device="cuda", dtype=torch.bfloat16)), positions,
                        half_freq, slots, cache2, heads, kv_heads, head_dim, head_dim // 2)
    want2 = R.ref_rope(parts.sum(0).to(torch.bfloat16), positions, half_freq, heads, kv_heads, head_dim, head_dim // 2)
    close(got2[:, :q], want2[:, :q], torch.bfloat16)


def test_linear_defers_split_sums(K):
    from iitj_llm_coopt_b200.kernels import PartialSums
    x, w = rnd((8, 4096), torch.bfloat16, 134), rnd((512, 4096), torch.bfloat16, 135, 0.05)
    out = torch.zeros(8, 512, device="cuda", dtype=torch.bfloat16)
    got = K.linear(x, w, out, defer=True)
    assert isinstance(got, PartialSums) and got.splits > 1
    close(got.sum(), R.ref_linear(x, w), torch.bfloat16, 0.5)
    assert isinstance(K.linear(x, w, out), torch.Tensor)


# ---- the tcgen05 matrix product (bfloat16) ---------------------------------------------
@pytest.mark.parametrize("tokens", [1, 7, 16, 17, 40, 100, 129, 300, 600])
@pytest.mark.parametrize("n,k", [(128, 64), (200, 96), (320, 176), (1000, 264), (136, 4104)])
def test_gemm_tcgen05_shapes(K, tokens, n, k):
    x, w = rnd((tokens, k), torch.bfloat16, 100), rnd((n, k), torch.bfloat16, 101, 0.05)
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.zeros(tokens, n, device="cuda", dtype=out_dtype)
        K.gemm_tcgen05(x, w, out)
        close(out, R.ref_linear(x, w), torch.bfloat16, 0.5 if out_dtype == torch.bfloat16 else 0.01)
    assert K.gemm_status() == 0


@pytest.mark.parametrize("tokens,n,k,splits", [(1, 128, 512, 2), (8, 320, 1024, 3), (33, 200, 4104, 9), (64, 136, 640, 16),
                                               (5, 256, 64, 4), (200, 384, 256, 2)])
def test_gemm_tcgen05_split_k(K, tokens, n, k, splits):
    x, w = rnd((tokens, k), torch.bfloat16, 102), rnd((n, k), torch.bfloat16, 103, 0.05)
    out = torch.zeros(tokens, n, device="cuda", dtype=torch.float32)
    K.gemm_tcgen05(x, w, out, splits=splits)
    close(out, R.ref_linear(x, w), torch.bfloat16, 0.01)
    assert K.gemm_status() == 0


@pytest.mark.parametrize("tokens,n,k,splits", [(1, 176, 64, 1), (9, 344, 96, 1), (70, 100, 200, 1), (8, 256, 1024, 4),
                                               (130, 384, 192, 1), (300, 1000, 264, 1), (16, 176, 4104, 7)])
def test_gemm_tcgen05_swiglu(K, tokens, n, k, splits):
    x, w = rnd((tokens, k), torch.bfloat16, 104), rnd((2 * n, k), torch.bfloat16, 105, 0.2)
    out = torch.zeros(tokens, n, device="cuda", dtype=torch.bfloat16)
    K.gemm_tcgen05(x, w, out, swiglu=True, splits=splits)
    close(out, R.ref_linear(x, w, swiglu=True), torch.bfloat16, 0.5)
    assert K.gemm_status() == 0


@pytest.mark.parametrize("tokens,n,k", [(1, 64, 64), (8, 192, 1024), (16, 448, 4104), (5, 1024, 200), (3, 14336, 4096),
                                        (17, 192, 264), (31, 448, 1024), (33, 64, 4104), (50, 1024, 200), (64, 14336, 4096),
                                        (65, 320, 136), (100, 192, 520), (128, 448, 1032)])
def test_gemm_tcgen05_swiglu_half_tiles(K, tokens, n, k):
    """The SwiGLU product of up to 128 tokens with 64 gate rows and 64 up rows in one 128-row MMA tile (token tiles of
    16, 32, 64 and 128; the up rows change hands 16 tokens at a time)."""
    x, w = rnd((tokens, k), torch.bfloat16, 304), rnd((2 * n, k), torch.bfloat16, 305, 0.2)
    for kb in (0, 100, 66):
        out = torch.full((tokens, n), float("nan"), device="cuda", dtype=torch.bfloat16)
        before = K.launches
        K.gemm_tcgen05(x, w, out, swiglu=True, smem_kb=kb, half=True)
        assert K.launches - before == 1
        close(out, R.ref_linear(x, w, swiglu=True), torch.bfloat16, 0.5)
    assert K.gemm_status() == 0
    with pytest.raises(Exception):
        K.gemm_tcgen05(rnd((129, k), torch.bfloat16, 1), w, torch.zeros(129, n, device="cuda", dtype=torch.bfloat16), swiglu=True, half=True)


def test_gemm_tcgen05_row_does_not_depend_on_batch(K):
    """With the same split count a token's row is bitwise the same alone and among others."""
    x, w = rnd((50, 264), torch.bfloat16, 106), rnd((200, 264), torch.bfloat16, 107, 0.05)
    full = torch.zeros(50, 200, device="cuda", dtype=torch.float32)
    one = torch.zeros(1, 200, device="cuda", dtype=torch.float32)
    K.gemm_tcgen05(x, w, full, splits=2)
    K.gemm_tcgen05(x[31:32].contiguous(), w, one, splits=2)
    assert torch.equal(full[31:32], one)


# ---- the persistent CTA-pair matrix product for many tokens (bfloat16) -------------------
@pytest.mark.parametrize("tokens,n,k", [(256, 256, 64), (300, 264, 136), (513, 1000, 264), (1000, 520, 4104), (130, 72, 64)])
def test_gemm_pair_shapes(K, tokens, n, k):
    x, w = rnd((tokens, k), torch.bfloat16, 110), rnd((n, k), torch.bfloat16, 111, 0.05)
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((tokens, n), float("nan"), device="cuda", dtype=out_dtype)
        K.gemm_pair(x, w, out)
        close(out, R.ref_linear(x, w), torch.bfloat16, 0.5 if out_dtype == torch.bfloat16 else 0.01)
    assert K.gemm_pair_status() == 0


@pytest.mark.parametrize("tokens,n,k", [(256, 128, 128), (300, 176, 72), (700, 1000, 264), (1030, 344, 2056)])
def test_gemm_pair_swiglu(K, tokens, n, k):
    x, w = rnd((tokens, k), torch.bfloat16, 112), rnd((2 * n, k), torch.bfloat16, 113, 0.2)
    out = torch.full((tokens, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    K.gemm_pair(x, w, out, swiglu=True)
    close(out, R.ref_linear(x, w, swiglu=True), torch.bfloat16, 0.5)
    assert K.gemm_pair_status() == 0


@pytest.mark.parametrize("tokens,n,k,swiglu", [(300, 600, 8200, False), (1200, 520, 8192, False), (520, 300, 9000, True)])
def test_gemm_pair_tail_split(K, tokens, n, k, swiglu):
    """Few tiles and a long k: every tile is cut along k over many clusters, whose partial sums the tile's
    first cluster adds.  Three launches in a row: the counters must be back at zero after each."""
    x, w = rnd((tokens, k), torch.bfloat16, 114), rnd(((2 if swiglu else 1) * n, k), torch.bfloat16, 115, 0.05)
    want = R.ref_linear(x, w, swiglu=swiglu)
    for _ in range(3):
        out = torch.full((tokens, n), float("nan"), device="cuda", dtype=torch.bfloat16)
        K.gemm_pair(x, w, out, swiglu=swiglu, tail_split=True)
        close(out, want, torch.bfloat16, 0.5)
        assert int(K._pair_counters[x.device].abs().sum()) == 0
    whole = torch.empty_like(out)
    K.gemm_pair(x, w, whole, swiglu=swiglu, tail_split=False)
    close(whole, want, torch.bfloat16, 0.5)
    assert K.gemm_pair_status() == 0


# ---- the tcgen05 prefill attention (bfloat16, head sizes 64 and 128) ------------------------
@pytest.mark.parametrize("head_dim", [128, 64])
@pytest.mark.parametrize("heads,kv_heads,page,window", [(8, 2, 16, 0), (4, 1, 8, 0), (2, 2, 64, 0), (3, 1, 128, 0),
                                                        (4, 2, 16, 100), (4, 2, 32, 128), (16, 1, 16, 0)])
def test_attention_tcgen05_portions(K, heads, kv_heads, page, window, head_dim):
    """Portions of several 128-query tiles, starting at positions that are no multiple of 128, beside
    short ones; page sizes from 8 to 128.  Decoded tokens in the same call go to the decode kernel."""
    D = head_dim
    assert K.lib.llm_attention_tcgen05_supported(heads, kv_heads, D, page)
    lens, qlens = [700, 130, 391, 64, 900, 5], [300, 130, 129, 64, 1, 2]
    q, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, D, page, lens, qlens, 120)
    out = torch.zeros(q.shape[0], heads * D, device="cuda", dtype=torch.bfloat16)
    K.attention(q, cache, meta, out, heads, kv_heads, D, window=window)
    want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads, D, window)
    close(out, want, torch.bfloat16)
    assert K.attention_status() == 0
    # the mma.sync kernel gives the same to rounding
    old, K.attention_tcgen05 = K.attention_tcgen05, False
    try:
        meta.attention_plan = None
        out2 = torch.zeros_like(out)
        K.attention(q, cache, meta, out2, heads, kv_heads, D, window=window)
    finally:
        K.attention_tcgen05 = old
    close(out2, want, torch.bfloat16)


@pytest.mark.parametrize("head_dim", [128, 64])
def test_attention_tcgen05_far_key_and_page_edges(K, head_dim):
    """One key among 2000 stands out for every query of a 256-token portion; it sits on a page edge."""
    heads, kv_heads, page, L, n, D = 2, 1, 16, 2000, 256, head_dim
    for far in (0, 15, 16, 127, 128, 1743):
        q, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, D, page, [L], [n], 130 + far)
        cache.mul_(0.05)
        pg, off = int(meta.block_table[0, far // page]), far % page
        key = rnd((D,), torch.float32, 131)
        key = key / key.norm()
        cache[pg, 0, 0, off] = (key * 40.0).to(torch.bfloat16)
        cache[pg, 1, 0, off] = 3.0
        q[:, :heads * D] = (key * 12.0).to(torch.bfloat16).repeat(heads)        # every query points at that key
        out = torch.zeros(n, heads * D, device="cuda", dtype=torch.bfloat16)
        K.attention(q, cache, meta, out, heads, kv_heads, D)
        want = R.ref_paged_attention(q, cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads, D)
        close(out, want, torch.bfloat16)
        assert (out.float() - 3.0).abs().max() < 0.1
    assert K.attention_status() == 0


def test_attention_tcgen05_says_when_scores_outgrow_its_one_pass_range(K):
    """Tiles after a request's first are exponentiated against the reference of the tiles before them, in one pass.  A
    key whose score lies more than 2^100 above everything before it is beyond what that pass can mend afterwards: the
    kernel leaves code 9 in its status word (which the engine reads with every sampled token) instead of a silent
    wrong result.  The same key in the first tile, where two passes run, is found as usual (with IITJ_ATTN_ONE_PASS=0 in
    the environment two passes run everywhere and nothing is flagged)."""
    import os
    from iitj_llm_coopt_b200.kernels import KernelError
    if os.environ.get("IITJ_ATTN_ONE_PASS", "1")[:1] == "0":
        pytest.skip("two passes everywhere: nothing to flag")
    heads, kv_heads, page, L, n, D = 2, 1, 16, 2000, 256, 128
    key = rnd((D,), torch.float32, 141)
    key = key / key.norm()
    for far, flagged in ((1743, True), (5, False)):
        q, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, D, page, [L], [n], 140 + far)
        cache.mul_(0.05)
        pg, off = int(meta.block_table[0, far // page]), far % page
        cache[pg, 0, 0, off] = (key * 80.0).to(torch.bfloat16)          # 80 * 12 / sqrt(128) * log2(e) = 122 in the kernel's units
        cache[pg, 1, 0, off] = 3.0
        q[:, :heads * D] = (key * 12.0).to(torch.bfloat16).repeat(heads)
        out = torch.zeros(n, heads * D, device="cuda", dtype=torch.bfloat16)
        K.attention(q, cache, meta, out, heads, kv_heads, D)
        torch.cuda.synchronize()
        status = K.attention_status()
        if flagged:
            assert status >> 16 == 9, hex(status)
            with pytest.raises(KernelError, match="prefill attention"):
                K.check_health([0, 0, status, 0])
        else:
            assert status == 0
            assert (out.float() - 3.0).abs().max() < 0.1
    assert K.attention_status() == 0                                   # (reading clears the word)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page,window,splits", [
    (8, 2, 128, 16, 0, 3), (32, 8, 128, 16, 0, 6), (16, 1, 64, 16, 0, 1), (6, 2, 64, 8, 0, 8), (4, 4, 128, 32, 0, 2),
    (8, 2, 128, 16, 300, 4), (3, 1, 64, 4, 0, 5), (2, 1, 128, 64, 0, 2), (12, 4, 64, 32, 200, 3)])
def test_attention_decode_fused(K, decode_loads, heads, kv_heads, head_dim, page, window, splits):
    """Decode attention that takes the qkv product's partial sums: adds them, rotates, stores the token's key and
    value and attends.  Against the plain rotation, store and attention; the slot of each token holds a
    huge stale value beforehand, which must neither be read nor survive."""
    from iitj_llm_coopt_b200.kernels import PartialSums
    lens = [700, 300, 1000, 257, 64, 65, 1, 1500, 128, 129]
    _, cache, meta = _paged_case(torch.bfloat16, heads, kv_heads, head_dim, page, lens, [1] * len(lens), 170)
    tokens, width = len(lens), (heads + 2 * kv_heads) * head_dim
    parts = rnd((splits, tokens, width), torch.float32, 171, 0.6)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))).cuda()
    pos = meta.positions.long()
    slots = (meta.block_table[torch.arange(tokens, device="cuda"), pos // page].long() * page + pos % page).to(torch.int32)
    meta.slots = slots
    _poison_unwritten_slots(cache, meta, lens, page)
    cache[(slots // page).long(), :, :, (slots % page).long(), :] = 3.0e4          # stale: would swamp everything
    want_cache = cache.clone()
    roped = R.ref_rope(parts.sum(0), meta.positions, inv_freq, heads, kv_heads, head_dim, head_dim).to(torch.bfloat16)
    R.ref_store(want_cache, roped, slots, heads, kv_heads, head_dim)
    want = R.ref_paged_attention(roped, want_cache, meta.block_table, meta.token_request, meta.positions, heads, kv_heads,
                                 head_dim, window)
    cos = torch.empty(tokens, head_dim // 2, device="cuda", dtype=torch.float32)
    sin = torch.empty_like(cos)
    K.rope_tables(meta.positions, inv_freq, cos, sin)
    qkv = PartialSums(K, parts, torch.zeros(tokens, width, device="cuda", dtype=torch.bfloat16))
    assert K.can_fuse_decode(qkv, meta, cache, heads, kv_heads, head_dim)
    out = torch.empty(tokens, heads * head_dim, device="cuda", dtype=torch.bfloat16)
    K.attention_decode_fused(qkv, (cos, sin), slots, cache, meta, out, heads, kv_heads, head_dim, window=window)
    close(out, want, torch.bfloat16)
    seen = lambda c: torch.nan_to_num(c, nan=7.0)                 # (the unwritten slots are NaN before and after)
    close(seen(cache), seen(want_cache), torch.bfloat16)
    # the unfused route (rope_store, then attention) gives the same keys and values, bit for bit
    cache2 = want_cache.clone()
    cache2[(slots // page).long(), :, :, (slots % page).long(), :] = 3.0e4
    K.rope_store(PartialSums(K, parts, torch.zeros(tokens, width, device="cuda", dtype=torch.bfloat16)), meta.positions,
                 inv_freq, slots, cache2, heads, kv_heads, head_dim, head_dim, tables=(cos, sin))
    assert torch.equal(seen(cache2), seen(cache))
    assert K.decode_status() == 0


def test_attention_decode_fused_is_refused_for_mixed_steps(K):
    from iitj_llm_coopt_b200.kernels import PartialSums
    _, cache, meta = _paged_case(torch.bfloat16, 4, 2, 128, 16, [70, 33], [5, 1], 180)
    parts = rnd((2, 6, 8 * 128), torch.float32, 181)
    qkv = PartialSums(K, parts, torch.zeros(6, 8 * 128, device="cuda", dtype=torch.bfloat16))
    assert not K.can_fuse_decode(qkv, meta, cache, 4, 2, 128)
    assert not K.can_fuse_decode(qkv.out, meta, cache, 4, 2, 128)


def test_a_wait_that_runs_out_is_reported_and_the_library_goes_on(K):
    """A bounded wait that gives up: the status word says which code, the sampler refuses to hand out tokens that
    were computed while a kernel had given up, and the next ordinary product is right again."""
    from iitj_llm_coopt_b200.kernels import KernelError
    from iitj_llm_coopt_b200.sampling import Sampler
    K.check_health()
    K.wait_probe(2000)
    torch.cuda.synchronize()
    code = K.gemm_status()
    assert code >> 16 == 7 and K.gemm_status() == 0           # read once, then clear
    # the same through the path serving takes: the word travels with the sampled ids
    K.wait_probe(500)
    sampler = Sampler(K, 0, "cuda")
    logits = rnd((3, 1000), torch.float32, 400)
    with pytest.raises(KernelError, match="gave up"):
        sampler.sample(logits, [(0.0, 0, 0)] * 3)
    assert sampler.sample(logits, [(0.0, 0, 0)] * 3) == logits.argmax(-1).tolist()    # cleared by the report
    x, w = rnd((8, 512), torch.bfloat16, 401), rnd((256, 512), torch.bfloat16, 402, 0.05)
    out = torch.empty(8, 256, device="cuda", dtype=torch.bfloat16)
    K.gemm_tcgen05(x, w, out)
    close(out, R.ref_linear(x, w), torch.bfloat16)
    K.check_health()
