"""Toy architectures defined here, in the test: a mixer with state of its own, a feed-forward with
routing, another position encoding, a layer named twice in the run order, a call that reads
another call's cache, and layers with a window beside layers without.  They are registered,
built and stepped through the framework's registries alone; no file of the framework
knows about it.  Stepping in portions must give what whole prompts give."""
from dataclasses import dataclass

import pytest
import torch

from iitj_llm_coopt_b200 import EngineConfig, build_engine, parts
from iitj_llm_coopt_b200.config.registry import ARCHITECTURES, register_architecture
from iitj_llm_coopt_b200.engine import StepEntry
from iitj_llm_coopt_b200.config.specs import (CacheNeed, FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec,
                                              NormSpec, PositionSpec)
from iitj_llm_coopt_b200.models.base import Architecture
from iitj_llm_coopt_b200.parts.base import ParamSpec, Part

import replay_cases as cases
from helpers import rel_err, run_steps


class RunningMeanMixer(Part):
    """y_t = W . mean(x_0 .. x_t) of the request: the running sum and the count are the
    request's state (width + 1 floats), carried from one portion to the next."""

    def __init__(self, spec, kernels, dtype, position=None):
        self.spec, self.k, self.dtype, self.width = spec, kernels, dtype, spec.width
        self.w = None

    @classmethod
    def parameters(cls, spec):
        return {"w": ParamSpec((spec.width, spec.width))}

    @classmethod
    def cache_need(cls, spec):
        return CacheNeed(kind="state", state_shape=(spec.width + 1,), state_dtype="float32")

    def forward(self, ctx, x, call):
        _, state = ctx.cache.view(call.cache)                 # [max_requests, width + 1]
        means = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        row = 0
        for b, n in enumerate(ctx.query_lens):                # a portion's tokens in order, request by request
            slot = ctx.slots_host[b]                          # (the cache manager cleared the slot when the request was admitted)
            sums = state[slot, :-1] + torch.cumsum(x[row:row + n].float(), dim=0)
            counts = state[slot, -1] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
            means[row:row + n] = sums / counts.unsqueeze(1)
            if call.write:
                state[slot, :-1] = sums[-1]
                state[slot, -1] = counts[-1]
            row += n
        out = ctx.buffer("toy.out", (x.shape[0], self.width), self.dtype)
        return self.k.linear(means.to(self.dtype), self.w, out)


class Top1RoutedFeedForward(Part):
    """A feed-forward with routing, defined in the test: a float32 router picks one of `experts` small
    SwiGLU experts per token; y = p_top * expert(x).  Tokens are grouped by expert on the host."""

    def __init__(self, spec, kernels, dtype):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.router = self.gate_up = self.down = None

    @classmethod
    def parameters(cls, spec):
        e = spec.experts
        return {"router": ParamSpec((e, spec.width), kind="matrix"),
                "gate_up": ParamSpec((e * 2 * spec.inner, spec.width)),
                "down": ParamSpec((e * spec.width, spec.inner))}

    def forward(self, ctx, x):
        sp = self.spec
        logits = x.float() @ self.router.float().t()                       # router logits in float32
        probs = torch.softmax(logits, dim=-1)
        top_p, top_e = probs.max(dim=-1)
        out = ctx.buffer("toy.ffn", (x.shape[0], sp.width), self.dtype)
        out.zero_()
        for e in range(sp.experts):
            idx = (top_e == e).nonzero().squeeze(-1)
            if idx.numel() == 0:
                continue
            xe = x[idx].contiguous()
            act = torch.empty(idx.numel(), sp.inner, dtype=self.dtype, device=x.device)
            self.k.linear(xe, self.gate_up[e * 2 * sp.inner:(e + 1) * 2 * sp.inner], act, swiglu=True)
            ye = torch.empty(idx.numel(), sp.width, dtype=self.dtype, device=x.device)
            self.k.linear(act, self.down[e * sp.width:(e + 1) * sp.width], ye)
            out[idx] = (ye.float() * top_p[idx].unsqueeze(1)).to(self.dtype)
        return out


class LinearFrequencyRotary(Part):
    """Another position encoding, defined in the test: rotation with frequencies that fall off linearly
    instead of geometrically; it reuses the engine's rotate-and-store kernel with its own table."""

    def __init__(self, spec, kernels, dtype, device="cuda"):
        self.spec, self.k, self.head_dim, self.rotary_dim = spec, kernels, spec.head_dim, spec.rotary_dim
        half = spec.rotary_dim // 2
        self.inv_freq = (1.0 - torch.arange(half, dtype=torch.float32) / half).div(spec.theta).to(device)

    def encode_and_store(self, ctx, qkv, cache_view, slots, heads, kv_heads):
        self.k.rope_store(qkv, ctx.positions, self.inv_freq, slots, cache_view, heads, kv_heads, self.head_dim,
                          self.rotary_dim)


@dataclass
class ToyConfig:
    width: int = 64
    vocab: int = 200
    inner: int = 96

    def to_dict(self):
        return {"architectures": ["ToyStateLM"], "width": self.width, "vocab": self.vocab, "inner": self.inner}

    @classmethod
    def from_dict(cls, d):
        return cls(d["width"], d["vocab"], d["inner"])

    def model_spec(self):
        norm = NormSpec("rmsnorm", self.width, 1e-5)
        ff = FeedForwardSpec("swiglu", self.width, self.inner)
        pos = PositionSpec("rope", head_dim=16, rotary_dim=8, theta=10000.0)       # partial rotation
        attn = LayerSpec.of("prenorm", mixer=MixerSpec("attention", self.width, heads=4, kv_heads=2, head_dim=16, position=pos),
                            feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm)
        routed = FeedForwardSpec("top1_routed", self.width, 48, experts=3, experts_per_token=1)
        pos2 = PositionSpec("linear_rotary", head_dim=16, rotary_dim=16, theta=50.0)
        toy = LayerSpec.of("prenorm", mixer=MixerSpec("running_mean", self.width), feed_forward=routed, mixer_norm=norm,
                           feed_forward_norm=norm)
        attn2 = LayerSpec.of("prenorm", mixer=MixerSpec("attention", self.width, heads=2, kv_heads=1, head_dim=16, position=pos2),
                             feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm)
        order = (LayerCall(layer=0, cache=0), LayerCall(layer=1, cache=1),
                 LayerCall(layer=0, cache=2),                   # layer 0 a second time, with a cache entry of its own
                 LayerCall(layer=0, cache=0, write=False),      # and a third time, reading the first call's keys
                 LayerCall(layer=2, cache=3))                   # other head counts, another position encoding
        return ModelSpec(width=self.width, vocab=self.vocab, layers=(attn, toy, attn2), order=order, final_norm=norm,
                         tie_embeddings=True, max_position=4096)


class ToyArch(Architecture):
    name = "ToyStateLM"
    config_class = ToyConfig

    def checkpoint_name(self, path, piece):
        return path if piece is None else f"{path}.{piece}"


@pytest.fixture
def toy_registered():
    parts.register_mixer("running_mean", RunningMeanMixer)
    parts.register_feed_forward("top1_routed", Top1RoutedFeedForward)
    parts.register_position_encoding("linear_rotary", LinearFrequencyRotary)
    register_architecture(ToyArch())
    yield
    parts.MIXERS.pop("running_mean", None)
    parts.FEED_FORWARDS.pop("top1_routed", None)
    parts.POSITION_ENCODINGS.pop("linear_rotary", None)
    ARCHITECTURES.pop("ToyStateLM", None)


def _engine(device, dtype):
    kernels = None
    if device == "cpu":
        from torch_kernels import TorchKernels
        kernels = TorchKernels()
    ec = EngineConfig(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=3, device=device)
    return build_engine(None, ec, config=ToyConfig(), architecture=ToyArch(), random_seed=3, kernels=kernels)


@pytest.mark.parametrize("device,dtype", [("cpu", "float32"),
                                          pytest.param("cuda:0", "float32", marks=pytest.mark.gpu),
                                          pytest.param("cuda:0", "bfloat16", marks=pytest.mark.gpu)])
def test_toy_mixer_with_state_steps_like_whole_prompts(toy_registered, device, dtype):
    eng = _engine(device, dtype)
    groups = eng.cache.groups
    assert len(groups) == 3 and len(eng.cache.paged) == 2             # two attention geometries, one state group
    assert groups[eng.cache.entry_group[1][0]].storage.shape == (1, 3 + 1, 65)        # three request slots and the padding slot
    assert eng.cache.entry_group[0][0] == eng.cache.entry_group[2][0] != eng.cache.entry_group[3][0]
    reqs = cases.requests_for(200, [50, 23, 70, 9], seed=4)
    whole = run_steps(eng, cases.whole(reqs))
    tol = 1e-4 if dtype == "float32" else 3e-2
    for label, steps in (("portions", cases.portions(reqs)), ("mixed", cases.mixed(reqs, live=3, seed=2)[0])):
        rows = run_steps(eng, steps)
        worst = max(rel_err(rows[k], whole[k]) for k in whole)
        assert worst <= tol, (label, worst)
        eng.cache.check()
    # the state matters: without the carried sum a later portion would differ
    a = run_steps(eng, [([("x", reqs["r0"][:20], [])], []), ([("x", reqs["r0"][20:30], list(range(10)))], ["x"])])
    b = run_steps(eng, [([("y", reqs["r0"][20:30], list(range(10)))], ["y"])])
    assert rel_err(a[("x", 25)], whole[("r0", 25)]) <= tol
    assert rel_err(b[("y", 5)], whole[("r0", 25)]) > 10 * tol


def test_unknown_part_kinds_are_clear_errors():
    spec = ToyConfig().model_spec()
    from iitj_llm_coopt_b200.models.decoder import model_parameter_specs
    with pytest.raises(KeyError) as e:
        model_parameter_specs(spec)
    assert "running_mean" in str(e.value) and "attention" in str(e.value)


# ---- a toy with a window: layers that keep every key beside layers that keep the last 20 ---------------
@dataclass
class ToyWindowConfig:
    head_dim: int = 16
    window: int = 20
    width: int = 64
    vocab: int = 200

    def to_dict(self):
        return {"architectures": ["ToyWindowLM"], "head_dim": self.head_dim, "window": self.window, "width": self.width,
                "vocab": self.vocab}

    @classmethod
    def from_dict(cls, d):
        return cls(d["head_dim"], d["window"], d["width"], d["vocab"])

    def model_spec(self):
        norm = NormSpec("rmsnorm", self.width, 1e-5)
        ff = FeedForwardSpec("swiglu", self.width, 96)
        pos = PositionSpec("rope", head_dim=self.head_dim, rotary_dim=self.head_dim, theta=10000.0)
        full = LayerSpec.of("prenorm", mixer=MixerSpec("attention", self.width, heads=4, kv_heads=2, head_dim=self.head_dim,
                                                       position=pos), feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm)
        near = LayerSpec.of("prenorm", mixer=MixerSpec("attention", self.width, heads=4, kv_heads=2, head_dim=self.head_dim,
                                                       window=self.window, position=pos), feed_forward=ff, mixer_norm=norm,
                            feed_forward_norm=norm)
        order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(1, 3))
        return ModelSpec(width=self.width, vocab=self.vocab, layers=(full, near), order=order, final_norm=norm,
                         tie_embeddings=True, max_position=4096)


class ToyWindowArch(Architecture):
    name = "ToyWindowLM"
    config_class = ToyWindowConfig

    def checkpoint_name(self, path, piece):
        return path if piece is None else f"{path}.{piece}"


def _window_engine(device, dtype, head_dim, window, pages=48, **options):
    kernels = None
    if device == "cpu":
        from torch_kernels import TorchKernels
        kernels = TorchKernels()
    ec = EngineConfig(dtype=dtype, page_size=8, num_pages=pages, max_num_seqs=3, device=device, **options)
    return build_engine(None, ec, config=ToyWindowConfig(head_dim, window), architecture=ToyWindowArch(), random_seed=5,
                        kernels=kernels)


@pytest.mark.parametrize("device,dtype,head_dim", [("cpu", "float32", 16),
                                                   pytest.param("cuda:0", "float32", 16, marks=pytest.mark.gpu),
                                                   pytest.param("cuda:0", "bfloat16", 16, marks=pytest.mark.gpu),
                                                   pytest.param("cuda:0", "bfloat16", 64, marks=pytest.mark.gpu),
                                                   pytest.param("cuda:0", "bfloat16", 128, marks=pytest.mark.gpu)])
def test_layers_with_a_window_beside_layers_without(device, dtype, head_dim):
    """Two cache groups with pages of their own: the windowed one gives pages back while a request lives, and every
    way of cutting gives what whole prompts give; a window changes nothing before position `window` and something
    after it."""
    window = 20
    eng = _window_engine(device, dtype, head_dim, window)
    cache = eng.cache
    assert len(cache.paged) == 2 and cache.windowed
    g_full, g_near = cache.entry_group[0][0], cache.entry_group[1][0]
    assert g_full != g_near and cache.entry_group[2][0] == g_full and cache.entry_group[3][0] == g_near
    reqs = cases.requests_for(200, [50, 23, 150, 9], seed=6)
    whole = run_steps(eng, cases.whole(reqs))
    tol = 1e-4 if dtype == "float32" else 3e-2
    for label, steps in (("last32", cases.last_one_by_one(reqs)), ("portions", cases.portions(reqs)),
                         ("mixed", cases.mixed(reqs, live=3, seed=2)[0])):
        rows = run_steps(eng, steps)
        worst = max(rel_err(rows[k], whole[k]) for k in whole)
        assert worst <= tol, (label, worst)
        cache.check()
        assert cache.groups[g_full].pool.num_free == 48 and cache.groups[g_near].pool.num_free == 48
    # pages of the windowed group come back while the request lives: 150 tokens hold 19 pages where every key is
    # kept, and never more than the window and one portion need where it is not
    toks, most_near = reqs["r2"], 0
    cache.admit("long")
    for i in range(0, 150, 10):
        eng.runner.step([StepEntry("long", toks[i:i + 10], [])])
        most_near = max(most_near, 48 - cache.groups[g_near].pool.num_free)
        cache.check()
    assert 48 - cache.groups[g_full].pool.num_free == 19
    assert most_near <= -(-(window + 10) // 8) + 1
    cache.release("long")
    # the window itself: the same weights without a window agree up to position 19 and not after
    everything = _window_engine(device, dtype, head_dim, 0)
    other = run_steps(everything, cases.whole({"r2": reqs["r2"]}))
    assert max(rel_err(other[("r2", p)], whole[("r2", p)]) for p in range(window)) <= tol
    assert rel_err(other[("r2", 140)], whole[("r2", 140)]) > 3 * tol


@pytest.mark.parametrize("device,dtype", [("cpu", "float32"), pytest.param("cuda:0", "bfloat16", marks=pytest.mark.gpu)])
def test_a_windowed_group_has_a_smaller_pool_than_the_full_one(device, dtype):
    """With the most tokens a step brings known (32), the windowed group's pool holds what three requests' windows and
    one step's tokens need, not whole contexts: fewer pages, less storage.  Replay within that bound agrees with
    whole prompts computed over roomy pools, and so does generation through the scheduler under that token budget."""
    window = 20
    small = _window_engine(device, dtype, 16, window, pages=48, max_num_batched_tokens=32)
    cache = small.cache
    g_full, g_near = cache.entry_group[0][0], cache.entry_group[1][0]
    want_pages = 3 * (-(-window // 8) + 2) + 32 // 8 + 3
    assert cache.groups[g_full].pool.num_pages == 48 and cache.groups[g_near].pool.num_pages == want_pages < 48
    if cache.groups[g_near].storage is not None:
        assert cache.groups[g_near].storage.shape[1] == want_pages + 1 and cache.groups[g_full].storage.shape[1] == 49
    assert cache.capacity_tokens == 48 * 8
    from iitj_llm_coopt_b200.cache import CacheManager
    from iitj_llm_coopt_b200.models.decoder import cache_needs
    needs = cache_needs(small.model_spec)
    itemsize = 4 if dtype == "float32" else 2
    per_entry = 2 * 2 * 16 * 8 * itemsize
    assert CacheManager.bytes_for(needs, 8, 48, itemsize, 3, 32) == 2 * per_entry * 49 + 2 * per_entry * (want_pages + 1)
    assert CacheManager.pages_for_bytes(needs, 8, CacheManager.bytes_for(needs, 8, 48, itemsize, 3, 32), itemsize, 3, 32) == 48
    roomy = _window_engine(device, dtype, 16, window, pages=48)
    reqs = cases.requests_for(200, [50, 23, 150, 9], seed=6)
    whole = run_steps(roomy, cases.whole(reqs))
    tol = 1e-4 if dtype == "float32" else 3e-2
    steps, _ = cases.mixed(reqs, live=2, seed=3, sizes=[7, 2, 13, 2, 5, 3, 16])        # at most 16 + 16 tokens a step
    rows = run_steps(small, steps)
    assert max(rel_err(rows[k], whole[k]) for k in whole) <= tol
    cache.check()
    assert cache.groups[g_near].pool.num_free == want_pages and cache.groups[g_full].pool.num_free == 48
    # through the scheduler: the token budget keeps every step within what the small pool was sized for
    outs = {}
    for name, eng in (("small", small), ("roomy", roomy)):
        seqs = [eng.new_sequence(toks[:40], 30, 0.0, True) for toks in list(reqs.values())[:3]]
        eng.run_until_done()
        outs[name] = [s.tokens[s.prompt_len:] for s in seqs]
        assert all(s.finish_reason == "length" for s in seqs)
        eng.cache.check()
    if dtype == "float32":
        assert outs["small"] == outs["roomy"]
    assert small.counters["num_preemptions_total"] == 0


# ---- a layer of five parts: norms after the mixer as well as before it -----------------------------------------
class PostNormBlock(parts.Arrangement):
    """x = mixer_norm(residual += delta); a = mixer_post_norm(mixer(x)); x = feed_forward_norm(residual += a);
    delta_out = feed_forward(x).  Five parts; the arrangement is defined here, in the test."""
    PARTS = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward"}

    def forward(self, ctx, residual, delta, call):
        from iitj_llm_coopt_b200.kernels import materialize
        from iitj_llm_coopt_b200.parts.base import delta_for
        x = self.mixer_norm.forward(ctx, residual, delta_for(self.mixer_norm, delta))
        a = materialize(self.mixer.forward(ctx, x, call))
        a = self.mixer_post_norm.forward(ctx, a.float().contiguous())          # a norm over the mixer's output alone
        x = self.feed_forward_norm.forward(ctx, residual, a)
        return residual, self.feed_forward.forward(ctx, x)


@dataclass
class ToyPostNormConfig:
    width: int = 64
    vocab: int = 200

    def to_dict(self):
        return {"architectures": ["ToyPostNormLM"], "width": self.width, "vocab": self.vocab}

    @classmethod
    def from_dict(cls, d):
        return cls(d["width"], d["vocab"])

    def model_spec(self):
        norm = NormSpec("rmsnorm", self.width, 1e-5)
        ff = FeedForwardSpec("swiglu", self.width, 96)
        pos = PositionSpec("rope", head_dim=16, rotary_dim=16, theta=10000.0)
        mixer = MixerSpec("attention", self.width, heads=4, kv_heads=2, head_dim=16, position=pos)
        five = LayerSpec.of("postnorm", mixer_norm=norm, mixer=mixer, mixer_post_norm=norm, feed_forward_norm=norm,
                            feed_forward=ff)
        four = LayerSpec.of("prenorm", mixer_norm=norm, mixer=mixer, feed_forward_norm=norm, feed_forward=ff)
        return ModelSpec(width=self.width, vocab=self.vocab, layers=(five, four), order=(LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2)),
                         final_norm=norm, tie_embeddings=False, max_position=4096)


class ToyPostNormArch(Architecture):
    name = "ToyPostNormLM"
    config_class = ToyPostNormConfig

    def checkpoint_name(self, path, piece):
        return path if piece is None else f"{path}.{piece}"


@pytest.mark.parametrize("device,dtype", [("cpu", "float32"), pytest.param("cuda:0", "float32", marks=pytest.mark.gpu),
                                          pytest.param("cuda:0", "bfloat16", marks=pytest.mark.gpu)])
def test_a_layer_of_five_parts_is_described_and_built(device, dtype):
    """An arrangement with another set of parts than the built-in one: registered from here, described by a LayerSpec
    that names five parts, built, loaded (each part's parameters under its own name) and stepped."""
    parts.register_arrangement("postnorm", PostNormBlock)
    try:
        kernels = None
        if device == "cpu":
            from torch_kernels import TorchKernels
            kernels = TorchKernels()
        ec = EngineConfig(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=3, device=device)
        eng = build_engine(None, ec, config=ToyPostNormConfig(), architecture=ToyPostNormArch(), random_seed=8, kernels=kernels)
        from iitj_llm_coopt_b200.models.decoder import model_parameter_specs
        names = model_parameter_specs(eng.model_spec)
        assert "layers.0.mixer_post_norm.weight" in names and "layers.1.mixer_post_norm.weight" not in names
        assert "lm_head.weight" in names
        block = eng.runner.model.layers[0]
        assert sorted(block.parts()) == sorted(PostNormBlock.PARTS) and block.mixer_post_norm is not block.mixer_norm
        reqs = cases.requests_for(200, [50, 23, 70, 9], seed=9)
        whole = run_steps(eng, cases.whole(reqs))
        tol = 1e-4 if dtype == "float32" else 3e-2
        for steps in (cases.portions(reqs), cases.mixed(reqs, live=3, seed=2)[0]):
            rows = run_steps(eng, steps)
            assert max(rel_err(rows[k], whole[k]) for k in whole) <= tol
        # the fifth part does something: with its gains turned round and tripled the logits move
        block.mixer_post_norm.weight.mul_(-3.0)
        moved = run_steps(eng, cases.whole({"r1": reqs["r1"]}))
        effect = rel_err(moved[("r1", 20)], whole[("r1", 20)])
        print("effect of the fifth part:", effect)
        assert effect > 0.1
    finally:
        parts.ARRANGEMENTS.pop("postnorm", None)


def test_a_layer_that_lacks_a_part_of_its_arrangement_is_a_clear_error():
    from iitj_llm_coopt_b200.models.decoder import model_parameter_specs
    norm = NormSpec("rmsnorm", 64, 1e-5)
    layer = LayerSpec.of("prenorm", mixer_norm=norm, feed_forward_norm=norm, feed_forward=FeedForwardSpec("swiglu", 64, 96))
    spec = ModelSpec(width=64, vocab=100, layers=(layer,), order=(LayerCall(0, 0),), final_norm=norm, tie_embeddings=True,
                     max_position=128)
    with pytest.raises(KeyError) as e:
        model_parameter_specs(spec)
    assert "mixer" in str(e.value) and "prenorm" in str(e.value)
