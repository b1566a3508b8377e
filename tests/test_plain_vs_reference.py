"""The plain implementation against outputs of the reference's own model code
(tests/golden/, made by tests/golden/make_golden.py on the CPU)."""
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_llama as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_logits(model_dirs, name):
    gold = load_file(os.path.join(GOLDEN, f"tiny_{name}.safetensors"))
    cfg, w = plain.read_model_dir(model_dirs[name], torch.float32)
    tokens = gold["tokens"].tolist()
    logits = plain.forward(cfg, w, tokens)
    ref = gold["logits"]
    assert logits.shape == ref.shape
    err = (logits - ref).abs().max().item() / ref.abs().max().item()
    assert err < 1e-5, err
    assert torch.equal(plain.inverse_frequencies(cfg), gold["inv_freq"])


def test_llama3_scaling_has_all_three_bands():
    from configs import TINY_B
    cfg = dict(TINY_B)
    inv = plain.inverse_frequencies(cfg)
    base = plain.inverse_frequencies({**cfg, "rope_scaling": None})
    ratio = (inv / base)
    assert (ratio == 1).any() and torch.isclose(ratio, torch.tensor(1 / 8.0)).any()
    assert ((ratio < 0.999) & (ratio > 1 / 8.0 + 1e-3)).any()


def test_greedy_generate_is_deterministic(model_dirs):
    cfg, w = plain.read_model_dir(model_dirs["A"], torch.float32)
    a = plain.greedy_generate(cfg, w, [5, 17, 3], 6)
    b = plain.greedy_generate(cfg, w, [5, 17, 3], 6)
    assert a == b and len(a) == 6


@pytest.mark.parametrize("heads,kv_heads,head_dim,tokens", [(4, 2, 16, 33), (3, 1, 32, 40), (6, 2, 64, 50), (32, 8, 128, 70)])
def test_plain_attention_is_pytorchs_grouped_causal_attention(heads, kv_heads, head_dim, tokens):
    """The reference hands attention to an external kernel (engine/model.py:204-207), so the reference's own code
    cannot anchor `plain.causal_attention`.  PyTorch's scaled_dot_product_attention with is_causal and enable_gqa is
    an independent statement of grouped causal attention (query head g reads key/value head g // (H / Hkv), keys
    0..t, scale 1/sqrt(D)): the head and group shapes of tiny A, tiny B, tiny C and the benchmark model."""
    g = torch.Generator().manual_seed(heads * 1000 + tokens)
    q = torch.randn(tokens, heads, head_dim, generator=g)
    k = torch.randn(tokens, kv_heads, head_dim, generator=g)
    v = torch.randn(tokens, kv_heads, head_dim, generator=g)
    ours = plain.causal_attention(q, k, v, 1.0 / head_dim ** 0.5)
    theirs = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0),
        is_causal=True, enable_gqa=True)[0].transpose(0, 1)
    assert (ours - theirs).abs().max().item() < 2e-6 * theirs.abs().max().item() + 2e-6
