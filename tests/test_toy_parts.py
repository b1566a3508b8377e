"""A toy architecture defined here, in the test: a mixer with state of its own, a feed-forward with
routing, another position encoding, a layer named twice in the run order, and a call that reads
another call's cache.  It is registered,
built and stepped through the framework's registries alone; no file of the framework
knows about it.  Stepping in portions must give what whole prompts give."""
from dataclasses import dataclass

import pytest
import torch

from iitj_llm_coopt_b200 import EngineConfig, build_engine, parts
from iitj_llm_coopt_b200.config.registry import ARCHITECTURES, register_architecture
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
            slot = ctx.slots_host[b]
            if ctx.starts[b] == 0:
                state[slot].zero_()
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
        attn = LayerSpec("prenorm", MixerSpec("attention", self.width, heads=4, kv_heads=2, head_dim=16, position=pos),
                         ff, norm, norm)
        routed = FeedForwardSpec("top1_routed", self.width, 48, experts=3, experts_per_token=1)
        pos2 = PositionSpec("linear_rotary", head_dim=16, rotary_dim=16, theta=50.0)
        toy = LayerSpec("prenorm", MixerSpec("running_mean", self.width), routed, norm, norm)
        attn2 = LayerSpec("prenorm", MixerSpec("attention", self.width, heads=2, kv_heads=1, head_dim=16, position=pos2),
                          ff, norm, norm)
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
