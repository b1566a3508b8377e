"""Each part of a layer alone (norm, position encoding, mixer, feed-forward, block, embedding
and head), built from its spec record at sizes other than the test models', run on a
step context made by the real step function, against the plain implementation's functions."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_llama as plain
from iitj_llm_coopt_b200 import kernels as kernels_mod, parts
from iitj_llm_coopt_b200.cache import CacheManager
from iitj_llm_coopt_b200.config.specs import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerCall, MixerSpec, NormSpec,
                                              PositionSpec)
from iitj_llm_coopt_b200.engine import ModelRunner, StepEntry

pytestmark = pytest.mark.gpu
DT = {"float32": (torch.float32, 2e-5), "bfloat16": (torch.bfloat16, 2e-2)}


def rnd(shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * std


def run_on_context(fn, needs, tokens_per_request, dtype, page=8, vocab=1000):
    """Calls fn(ctx) inside a real step: the runner builds the flattened batch and the cache."""
    cache = CacheManager(needs, page, 64, max_requests=8, dtype=dtype, device="cuda:0")
    model = SimpleNamespace(spec=SimpleNamespace(vocab=vocab), forward=fn)
    runner = ModelRunner(model, cache, "cuda:0")
    entries = []
    for i, n in enumerate(tokens_per_request):
        cache.admit(i)
        entries.append(StepEntry(i, list(range(n)), [n - 1]))
    return runner.step(entries), runner, cache


def err(got, want):
    return (got.float().cpu() - want.float()).abs().max().item() / want.float().abs().max().item()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    dt, tol = DT[dtype]
    K = kernels_mod.load()
    width, eps = 200, 3e-6
    norm = parts.NORMS["rmsnorm"](NormSpec("rmsnorm", width, eps), K, dt)
    assert list(parts.RMSNorm.parameters(norm.spec)) == ["weight"]
    w = 1 + 0.1 * rnd((width,), 1)
    norm.load({"weight": w.to(dt).cuda()})
    x = rnd((7, width), 2, 3.0)

    def fn(ctx):
        return norm.forward(ctx, x.cuda().clone()).clone()
    got, _, _ = run_on_context(fn, [], [7], dt)
    assert err(got, plain.rms_norm(x, w.to(dt).float(), eps)) <= tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("scaled", [False, True])
def test_rotary_part(dtype, scaled):
    dt, tol = DT[dtype]
    K = kernels_mod.load()
    heads, kv_heads, D = 3, 1, 48
    scaling = (("factor", 8.0), ("high_freq_factor", 4.0), ("low_freq_factor", 1.0),
               ("original_max_position_embeddings", 64), ("rope_type", "llama3")) if scaled else ()
    rope = parts.POSITION_ENCODINGS["rope"](PositionSpec("rope", D, D, 500000.0, scaling), K, dt)
    cfg = {"head_dim": D, "rope_theta": 500000.0, "rope_scaling": dict(scaling) or None}
    assert torch.allclose(rope.inv_freq.cpu(), plain.inverse_frequencies(cfg), rtol=1e-6, atol=0)
    n = 40
    qkv = rnd((n, (heads + 2 * kv_heads) * D), 3).to(dt)

    def fn(ctx):
        buf = qkv.cuda().clone()
        rope.encode_and_store(ctx, buf, None, None, heads, kv_heads)
        return buf
    got, _, _ = run_on_context(fn, [], [n], dt)
    cos, sin = plain.rope_tables(cfg, n)
    want_q = plain.apply_rope(qkv[:, :heads * D].float().view(n, heads, D), cos, sin).reshape(n, -1)
    assert err(got[:, :heads * D], want_q) <= tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_part(dtype):
    dt, tol = DT[dtype]
    K = kernels_mod.load()
    width, inner = 136, 344
    ff = parts.FEED_FORWARDS["swiglu"](FeedForwardSpec("swiglu", width, inner), K, dt)
    p = parts.SwiGLU.parameters(ff.spec)
    assert p["gate_up"].shape == (2 * inner, width) and p["gate_up"].pieces == (("gate", inner), ("up", inner))
    gate, up, down = rnd((inner, width), 4, 0.1).to(dt), rnd((inner, width), 5, 0.1).to(dt), rnd((width, inner), 6, 0.1).to(dt)
    ff.load({"gate_up": torch.cat([gate, up]).cuda(), "down": down.cuda()})
    x = rnd((9, width), 7).to(dt)

    def fn(ctx):
        return ff.forward(ctx, x.cuda()).clone()
    got, _, _ = run_on_context(fn, [], [9], dt)
    assert err(got, plain.swiglu(x.float(), gate.float(), up.float(), down.float())) <= tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,D", [(6, 3, 32), (4, 1, 64), (2, 2, 128)])
def test_attention_part(dtype, heads, kv_heads, D):
    """Two requests whole in one step: the mixer projects, rotates, stores and attends."""
    dt, tol = DT[dtype]
    K = kernels_mod.load()
    width = 120
    pos = PositionSpec("rope", D, D, 10000.0)
    spec = MixerSpec("attention", width, heads=heads, kv_heads=kv_heads, head_dim=D, position=pos)
    rope = parts.RotaryEmbedding(pos, K, dt)
    attn = parts.MIXERS["attention"](spec, K, dt, position=rope)
    wq, wk, wv = rnd((heads * D, width), 8, 0.1).to(dt), rnd((kv_heads * D, width), 9, 0.1).to(dt), rnd((kv_heads * D, width), 10, 0.1).to(dt)
    wo = rnd((width, heads * D), 11, 0.1).to(dt)
    attn.load({"qkv": torch.cat([wq, wk, wv]).cuda(), "o": wo.cuda()})
    lens = [37, 70]
    x = rnd((sum(lens), width), 12).to(dt)

    def fn(ctx):
        return attn.forward(ctx, x.cuda(), LayerCall(0, 0, True)).clone()
    got, _, cache = run_on_context(fn, [parts.PagedAttention.cache_need(spec)], lens, dt)
    cfg = {"head_dim": D, "rope_theta": 10000.0, "rope_scaling": None}
    row = 0
    for n in lens:
        xs = x[row:row + n].float()
        cos, sin = plain.rope_tables(cfg, n)
        q = plain.apply_rope((xs @ wq.float().t()).view(n, heads, D), cos, sin)
        k = plain.apply_rope((xs @ wk.float().t()).view(n, kv_heads, D), cos, sin)
        v = (xs @ wv.float().t()).view(n, kv_heads, D)
        want = plain.causal_attention(q, k, v, 1 / math.sqrt(D)).reshape(n, -1) @ wo.float().t()
        assert err(got[row:row + n], want) <= tol
        row += n
    cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    dt, tol = DT[dtype]
    K = kernels_mod.load()
    vocab, width = 333, 72
    table = rnd((vocab, width), 13).to(dt)
    emb = parts.EMBEDDINGS["table"](EmbeddingSpec("table", vocab, width), K, dt)
    head = parts.HEADS["linear"](HeadSpec("linear", vocab, width, scale=0.5), K, dt)
    emb.load({"weight": table.cuda()})
    head.load({"weight": table.cuda()})

    def fn(ctx):
        res = emb.forward(ctx)
        return res.clone(), head.forward(ctx, res.to(dt)).clone()
    (res, logits), _, _ = run_on_context(fn, [], [5], dt, vocab=vocab)
    assert torch.equal(res.cpu(), table[:5].float())
    assert logits.dtype == torch.float32
    assert err(logits, 0.5 * (table[:5].float() @ table.float().t())) <= tol
