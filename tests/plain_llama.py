"""A plain, slow Llama: whole sequences, no cache, no batching, one function per part.

Written from the formulas of the reference engine (mohsinmubarak/iitj-llm-coopt); each
function cites the lines it restates.  It shares no code with the engine under test: it
reads config.json and the safetensors file itself and uses only elementary torch ops.
tests/golden/ holds outputs of the reference's own model code for two tiny models, and
tests/test_plain_vs_reference.py checks this file against them.
"""
import glob
import json
import math
import os

import torch
from safetensors import safe_open


def read_model_dir(model_dir, dtype=torch.float32, device="cpu"):
    """(config dict, {tensor name: tensor as `dtype`}) -- engine/model.py:137-142.  Every *.safetensors file of the
    folder is read (engine/model.py:139).  `device`: where the tensors are put; `forward` computes where they lie (a
    GPU only for models too large for the CPU; the formulas are the same elementary torch ops)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])  # engine/model.py:47
    weights = {}
    for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
        with safe_open(path, framework="pt", device="cpu") as sf:
            for name in sf.keys():
                weights[name] = sf.get_tensor(name).to(device=device, dtype=dtype)
    return cfg, weights


def inverse_frequencies(cfg):
    """engine/model.py:68-82 (llama3_inv_freq)."""
    dim = cfg["head_dim"]
    inv_freq = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    rs = cfg.get("rope_scaling")
    if not rs or rs.get("rope_type") != "llama3":
        return inv_freq
    factor, lo, hi = rs["factor"], rs["low_freq_factor"], rs["high_freq_factor"]
    old = rs["original_max_position_embeddings"]
    low_wavelen, high_wavelen = old / lo, old / hi
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old / wavelen - lo) / (hi - lo)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    is_medium = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
    return torch.where(is_medium, smoothed, scaled)


def rope_tables(cfg, length):
    """cos, sin [length, head_dim] in float32 -- engine/model.py:119-124 (before its cast to the model dtype)."""
    pos = torch.arange(length, dtype=torch.float32)
    freqs = torch.outer(pos, inverse_frequencies(cfg))
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rms_norm(x, weight, eps):
    """engine/model.py:85-89."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * xf.to(x.dtype)


def rotate_half(x):
    """engine/model.py:92-94."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rope(x, cos, sin):
    """x [T, heads, D]; engine/model.py:187-188, 199-200."""
    return x * cos.unsqueeze(1) + rotate_half(x) * sin.unsqueeze(1)


def causal_attention(q, k, v, scale, window=0):
    """q [T, H, D], k, v [T, Hkv, D] of one whole sequence.  The reference hands this to an
    external kernel (engine/model.py:204-207: causal, softmax_scale = 1/sqrt(D), query head g
    reads kv head g // (H / Hkv)); softmax over keys 0..t for query t, in float32."""
    T, H, D = q.shape
    group = H // k.shape[1]
    kk = k.repeat_interleave(group, dim=1).float()
    vv = v.repeat_interleave(group, dim=1).float()
    scores = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    qpos = torch.arange(T, device=q.device).view(1, T, 1)
    kpos = torch.arange(T, device=q.device).view(1, 1, T)
    hidden = kpos > qpos
    if window > 0:
        hidden = hidden | (kpos < qpos - window + 1)
    scores = scores.masked_fill(hidden, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), vv).to(q.dtype)


def swiglu(x, gate_w, up_w, down_w):
    """engine/model.py:210-211."""
    gate = x @ gate_w.t()
    up = x @ up_w.t()
    return (torch.nn.functional.silu(gate) * up) @ down_w.t()


def forward(cfg, w, tokens, collect=None):
    """Logits [len(tokens), vocab] in float32 at every position of one whole sequence.
    Layer order as engine/model.py:191-213 (forward_reference)."""
    T = len(tokens)
    H, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    cos, sin = rope_tables(cfg, T)
    device = w["model.embed_tokens.weight"].device
    x = w["model.embed_tokens.weight"][torch.tensor(tokens, dtype=torch.long, device=device)]   # engine/model.py:191
    cos, sin = cos.to(device=device, dtype=x.dtype), sin.to(device=device, dtype=x.dtype)       # engine/model.py:123-124
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], eps)                         # :193
        q = (h @ w[p + "self_attn.q_proj.weight"].t()).view(T, H, D)                  # :194-198
        k = (h @ w[p + "self_attn.k_proj.weight"].t()).view(T, Hkv, D)
        v = (h @ w[p + "self_attn.v_proj.weight"].t()).view(T, Hkv, D)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)                       # :199-200
        attn = causal_attention(q, k, v, 1.0 / math.sqrt(D))                          # :102, 204-207
        x = x + attn.reshape(T, H * D) @ w[p + "self_attn.o_proj.weight"].t()         # :208
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)                # :209
        x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"])                                 # :210-211
        if collect is not None:
            collect.append(x.clone())
    x = rms_norm(x, w["model.norm.weight"], eps)                                      # :212
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]  # :106
    return (x @ head.t()).float()                                                     # :218


def greedy_generate(cfg, w, prompt, max_tokens, eos_ids=(), ignore_eos=True):
    """Greedy continuation by recomputing the whole sequence for every token
    (sampling rule engine/spec_decode.py:14-15, stop rules engine/engine.py:293-308)."""
    tokens = list(prompt)
    out = []
    for _ in range(max_tokens):
        nxt = int(forward(cfg, w, tokens)[-1].argmax())
        tokens.append(nxt)
        out.append(nxt)
        if not ignore_eos and nxt in eos_ids:
            break
    return out
