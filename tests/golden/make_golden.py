"""Makes tests/golden/*.safetensors: logits of the reference's own model code on CPU.

    python tests/golden/make_golden.py /path/to/reference

The reference's engine/model.py imports vllm's CUDA ops at import time, which cannot load
without a GPU driver, so three modules are replaced by stand-ins before the import:
`vllm`, `vllm._custom_ops` (unused by forward_reference) and `vllm.vllm_flash_attn`, whose
`flash_attn_varlen_func` is restated below in plain torch with the call's signature
(engine/model.py:204-207).  Everything else that produces the logits is the reference's own
code, unmodified: LlamaConfig, llama3_inv_freq, the RoPE tables and their application,
rms_norm, the QKV / gate-up fusion, the cache write by (page, offset), BlockManager's
tables and slot mapping, SwiGLU, residuals, final norm and the (tied) head.  Attention
itself is therefore anchored on the formula only.

For each tiny configuration the model folder is written with this repository's
random-weights mode (seeded), a fixed prompt is run whole (all logits), and the logits are
stored with the prompt.  tests/test_plain_vs_reference.py rebuilds the same folder and
compares tests/plain_llama.py with these files.
"""
import os
import sys
import tempfile
import types

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))


def paged_attention_stand_in(q, k, v, cu_seqlens_q, max_seqlen_q, seqused_k, max_seqlen_k, softmax_scale,
                             causal, block_table, fa_version=2):
    T, H, D = q.shape
    Hkv, bs = k.shape[2], k.shape[1]
    out = torch.empty_like(q)
    for b in range(len(seqused_k)):
        s, e = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        L, n = int(seqused_k[b]), e - s
        nb = -(-L // bs)
        blocks = block_table[b, :nb].long()
        kk = k[blocks].reshape(nb * bs, Hkv, D)[:L].float().repeat_interleave(H // Hkv, dim=1)
        vv = v[blocks].reshape(nb * bs, Hkv, D)[:L].float().repeat_interleave(H // Hkv, dim=1)
        sc = torch.einsum("qhd,khd->hqk", q[s:e].float(), kk) * softmax_scale
        qpos = torch.arange(L - n, L).view(1, n, 1)
        kpos = torch.arange(L).view(1, 1, L)
        sc = sc.masked_fill(kpos > qpos, float("-inf"))
        out[s:e] = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), vv).to(q.dtype)
    return out


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_DIR")
    if not ref or not os.path.isdir(ref):
        sys.exit("give the reference's checkout as the first argument or in $REFERENCE_DIR")
    fa = types.ModuleType("vllm.vllm_flash_attn")
    fa.flash_attn_varlen_func = paged_attention_stand_in
    ops = types.ModuleType("vllm._custom_ops")
    v = types.ModuleType("vllm")
    v.__path__ = []
    v._custom_ops, v.vllm_flash_attn = ops, fa
    sys.modules.update({"vllm": v, "vllm._custom_ops": ops, "vllm.vllm_flash_attn": fa})
    sys.path.insert(0, ref)
    import engine.model as M
    from engine.block_manager import BlockManager

    from configs import CONFIGS
    from iitj_llm_coopt_b200.weights import write_model_dir
    from plain_llama import read_model_dir

    for name, length in (("A", 33), ("B", 70)):
        cfg_dict, seed, page = CONFIGS[name]
        with tempfile.TemporaryDirectory() as d:
            write_model_dir(cfg_dict, d, seed)
            cfg = M.LlamaConfig.from_json(os.path.join(d, "config.json"))
            _, weights = read_model_dir(d, torch.float32)
        model = M.Llama(cfg, dict(weights), device="cpu", dtype=torch.float32)
        model.fused = False
        pages = -(-length // page) + 2
        shape = (pages, page, cfg.num_key_value_heads, cfg.head_dim)
        model.use_kv_views([torch.zeros(shape) for _ in range(cfg.num_hidden_layers)],
                           [torch.zeros(shape) for _ in range(cfg.num_hidden_layers)], page)
        bm = BlockManager(pages, page)
        g = torch.Generator().manual_seed(100 + seed)
        tokens = torch.randint(0, cfg.vocab_size, (length,), generator=g).tolist()
        bm.ensure(0, length)
        batch = M.Batch(input_ids=torch.tensor(tokens), positions=torch.arange(length),
                        cu_seqlens_q=torch.tensor([0, length], dtype=torch.int32),
                        seq_lens=torch.tensor([length], dtype=torch.int32),
                        block_table=bm.block_table_tensor([0]), slot_mapping=bm.slot_mapping(0, 0, length),
                        logits_indices=torch.arange(length), max_seqlen_q=length, max_seqlen_k=length)
        logits = model.forward(batch)
        inv_freq = M.llama3_inv_freq(cfg)
        out = os.path.join(HERE, f"tiny_{name}.safetensors")
        save_file({"tokens": torch.tensor(tokens, dtype=torch.int32), "logits": logits.float().contiguous(),
                   "inv_freq": inv_freq.float().contiguous()}, out)
        print(name, "->", out, tuple(logits.shape))


if __name__ == "__main__":
    main()
