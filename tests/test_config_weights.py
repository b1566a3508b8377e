"""Configuration, registry, weight loading errors and the random-weights mode (CPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from configs import TINY_A, TINY_B
from iitj_llm_coopt_b200.config import ConfigError, LlamaConfig, load_config
from iitj_llm_coopt_b200.config.registry import ARCHITECTURES, architecture_for
from iitj_llm_coopt_b200.models.decoder import cache_needs, model_parameter_specs
from iitj_llm_coopt_b200.weights import WeightError, load_parameters, write_model_dir


def test_config_reads_every_key():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (96, 256, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 1, 32)
    assert c.vocab_size == 320 and c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0
    assert c.rope_scaling["factor"] == 8.0 and c.tie_word_embeddings and c.eos_ids == (1, 2)
    assert c.max_position_embeddings == 512
    assert c.kv_bytes_per_token(2) == 2 * 3 * 1 * 32 * 2


def test_head_dim_defaults_to_hidden_over_heads():
    d = {k: v for k, v in TINY_A.items() if k != "head_dim"}
    assert LlamaConfig.from_dict(d).head_dim == 16


def test_rope_parameters_spelling_is_accepted():
    d = {k: v for k, v in TINY_B.items() if k not in ("rope_theta", "rope_scaling")}
    d["rope_parameters"] = {"rope_theta": 500000.0, **TINY_B["rope_scaling"]}
    c = LlamaConfig.from_dict(d)
    assert c.rope_theta == 500000.0 and c.rope_scaling["rope_type"] == "llama3"


@pytest.mark.parametrize("change,word", [
    ({"hidden_size": None}, "hidden_size"), ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 24}, "head_dim"),
    ({"attention_bias": True}, "bias"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2}}, "lacks"),
])
def test_bad_configs_are_refused(change, word):
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict({**TINY_A, **change})
    assert word in str(e.value)


def test_registry_picks_by_architecture_name():
    assert architecture_for(TINY_A).name == "LlamaForCausalLM"
    assert "LlamaForCausalLM" in ARCHITECTURES
    with pytest.raises(ConfigError) as e:
        architecture_for({**TINY_A, "architectures": ["NoSuchModel"]})
    assert "NoSuchModel" in str(e.value) and "LlamaForCausalLM" in str(e.value)


def test_model_spec_is_data():
    arch = architecture_for(TINY_B)
    spec = arch.model_spec(LlamaConfig.from_dict(TINY_B))
    assert len(spec.layers) == 3 and [c.layer for c in spec.order] == [0, 1, 2]
    assert all(c.cache == i and c.write for i, c in enumerate(spec.order))
    assert spec.layers[0].arrangement == "prenorm"
    assert spec.layers[0].names() == ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")
    m = spec.layers[0].part("mixer")
    assert (m.kind, m.heads, m.kv_heads, m.head_dim, m.window) == ("attention", 3, 1, 32, 0)
    assert m.position.kind == "rope" and dict(m.position.scaling)["factor"] == 8.0
    assert spec.layers[0].part("feed_forward").inner == 256 and spec.final_norm.eps == 1e-6
    assert (spec.embedding_spec().kind, spec.head_spec().kind, spec.head_spec().vocab) == ("table", "linear", 320)
    needs = cache_needs(spec)
    assert len(needs) == 3 and all(n.kind == "paged_kv" and n.kv_heads == 1 and n.head_dim == 32 for n in needs)
    names = model_parameter_specs(spec)
    assert "lm_head.weight" not in names and names["layers.2.mixer.qkv"].shape == (5 * 32, 96)


def test_random_model_dir_roundtrip(tmp_path):
    d = write_model_dir(TINY_A, str(tmp_path / "m"), seed=0)
    raw = json.load(open(os.path.join(d, "config.json")))
    assert raw["architectures"] == ["LlamaForCausalLM"] and raw["hidden_size"] == 64
    t = load_file(os.path.join(d, "model.safetensors"))
    assert t["model.layers.1.mlp.gate_proj.weight"].shape == (176, 64)
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert 0.015 < t["model.embed_tokens.weight"].float().std() < 0.025
    g = t["model.norm.weight"].float()
    assert 0.89 <= g.min() and g.max() <= 1.11          # bfloat16 rounding of 1 +- 0.1
    # same seed, same numbers; other seed, other numbers
    d2 = write_model_dir(TINY_A, str(tmp_path / "m2"), seed=0)
    d3 = write_model_dir(TINY_A, str(tmp_path / "m3"), seed=1)
    t2, t3 = load_file(os.path.join(d2, "model.safetensors")), load_file(os.path.join(d3, "model.safetensors"))
    assert all(torch.equal(t[k], t2[k]) for k in t)
    assert not torch.equal(t["lm_head.weight"], t3["lm_head.weight"])
    arch, cfg = load_config(d)
    spec = arch.model_spec(cfg)
    p = load_parameters(d, arch, cfg, spec, torch.bfloat16, device="cpu")
    assert p["layers.0.mixer.qkv"].dtype == torch.bfloat16 and p["layers.0.mixer.qkv"].shape == (128, 64)
    assert torch.equal(p["layers.0.mixer.qkv"][64:96], t["model.layers.0.self_attn.k_proj.weight"])
    assert torch.equal(p["layers.1.feed_forward.gate_up"][176:], t["model.layers.1.mlp.up_proj.weight"])
    p32 = load_parameters(d, arch, cfg, spec, torch.float32, device="cpu")
    assert all(v.dtype == torch.float32 for v in p32.values())
    assert torch.equal(p32["final_norm.weight"], t["model.norm.weight"].float())


def test_stored_float32_vectors_stay_float32_in_bfloat16_mode(tmp_path):
    d = write_model_dir(TINY_A, str(tmp_path / "m"), seed=0)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    t["model.norm.weight"] = t["model.norm.weight"].float() + 1e-4     # not representable in bfloat16
    t["model.layers.0.self_attn.o_proj.weight"] = t["model.layers.0.self_attn.o_proj.weight"].float()
    save_file(t, path)
    arch, cfg = load_config(d)
    p = load_parameters(d, arch, cfg, arch.model_spec(cfg), torch.bfloat16, device="cpu")
    assert p["final_norm.weight"].dtype == torch.float32 and torch.equal(p["final_norm.weight"], t["model.norm.weight"])
    assert p["layers.0.mixer.o"].dtype == torch.bfloat16              # matrices run in the engine's type


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_model_dir(TINY_A, str(tmp_path / "m"), seed=0)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.mlp.down_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    t["model.layers.0.extra.weight"] = torch.zeros(3)
    save_file(t, path)
    arch, cfg = load_config(d)
    with pytest.raises(WeightError) as e:
        load_parameters(d, arch, cfg, arch.model_spec(cfg), torch.float32, device="cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    text = str(err)
    for word in ("missing", "unexpected", "wrong shapes", "model.norm.weight", "extra.weight", "(16, 64)", "(32, 64)"):
        assert word in text


def test_tied_model_may_carry_an_unused_head(tmp_path):
    d = write_model_dir(TINY_B, str(tmp_path / "m"), seed=1)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    assert "lm_head.weight" not in t
    t["lm_head.weight"] = torch.zeros(320, 96, dtype=torch.bfloat16)
    save_file(t, path)
    arch, cfg = load_config(d)
    p = load_parameters(d, arch, cfg, arch.model_spec(cfg), torch.float32, device="cpu")
    assert "lm_head.weight" not in p


def test_missing_files_are_clear_errors(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, cfg = load_config(str(tmp_path))
    with pytest.raises(FileNotFoundError):
        load_parameters(str(tmp_path), arch, cfg, arch.model_spec(cfg), torch.float32, device="cpu")


def test_random_weights_command_line(tmp_path):
    """`python -m iitj_llm_coopt_b200.weights` writes a folder that the loader's checks accept and that is the
    same for the same seed."""
    import subprocess, sys
    from configs import TINY_B
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(TINY_B))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for name in ("a", "b"):
        subprocess.run([sys.executable, "-m", "iitj_llm_coopt_b200.weights", "--config", str(cfg_path), "--out",
                        str(tmp_path / name), "--seed", "5"], check=True, cwd=root, capture_output=True)
    from safetensors.torch import load_file
    a, b = load_file(str(tmp_path / "a" / "model.safetensors")), load_file(str(tmp_path / "b" / "model.safetensors"))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    assert "lm_head.weight" not in a and a["model.embed_tokens.weight"].shape == (TINY_B["vocab_size"], TINY_B["hidden_size"])
    assert json.load(open(tmp_path / "a" / "config.json"))["num_key_value_heads"] == TINY_B["num_key_value_heads"]
