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
