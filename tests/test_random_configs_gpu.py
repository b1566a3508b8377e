"""Random tiny configurations through the engine: head sizes in steps of 16 up to 256, any number of heads
and groups, widths, inner sizes and vocabularies that are no multiple of anything, with and without llama3
rotary scaling, tied and untied heads, page sizes from 4 to 64.  Each is replayed whole, with the last 32 tokens
one by one, in portions and mixed over a pool that is just large enough, in float32 and bfloat16, against the
plain implementation; every other checkpoint is stored in float32.  The configurations are drawn from fixed seeds, so a failure names its seed."""
import random

import pytest
import torch

import plain_llama as plain
import replay_cases as cases
from helpers import make_engine, rel_err, run_steps
from iitj_llm_coopt_b200.weights import write_model_dir

FP32_TOL, BF16_TOL = 1e-4, 2e-2


def random_config(rng):
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 128, 64, 144, 160, 192, 256])
    kv = rng.choice([1, 1, 2, 2, 3, 4, 5, 8])
    group = rng.choice([1, 1, 2, 3, 4, 5, 7, 8])
    while kv * group * head_dim > 2048:
        if group > 1:
            group -= 1
        elif kv > 1:
            kv -= 1
        else:
            break
    scaling = None
    if rng.random() < 0.5:
        scaling = {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0, 32.0]), "low_freq_factor": 1.0,
                   "high_freq_factor": rng.choice([2.0, 4.0]), "original_max_position_embeddings": rng.choice([32, 64, 256])}
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": rng.choice([rng.randrange(24, 400), rng.randrange(3, 60) * 8, rng.choice([64, 128, 256, 512])]),
        "intermediate_size": rng.choice([rng.randrange(20, 700), rng.randrange(3, 90) * 8, rng.choice([128, 256, 1024])]),
        "num_hidden_layers": rng.choice([1, 2, 2, 3]),
        "num_attention_heads": kv * group, "num_key_value_heads": kv, "head_dim": head_dim,
        "vocab_size": rng.choice([rng.randrange(17, 3000), rng.choice([256, 1024, 4096]), rng.randrange(100, 700)]),
        "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-5, 1e-4]), "rope_theta": rng.choice([10000.0, 500000.0, 1000.0, 1e6]),
        "rope_scaling": scaling, "tie_word_embeddings": rng.random() < 0.5, "max_position_embeddings": 4096,
        "eos_token_id": 1,
    }


@pytest.mark.gpu
@pytest.mark.parametrize("seed", list(range(100, 116)))
def test_random_configuration(tmp_path, seed):
    rng = random.Random(seed)
    cfg = random_config(rng)
    page = rng.choice([16, 16, 16, 8, 32, 64, 4])
    lens = [rng.choice([1, 2, 3, 5, 17, 33, 63, 64, 65, 100, 127, 128, 129, 130, 200, 257, 300])
            for _ in range(rng.choice([3, 4, 5]))]
    # every other checkpoint is stored in float32, with values that bfloat16 cannot hold: the float32 engine must use
    # them as they are, the bfloat16 engine rounds the matrices and keeps the norm gains
    write_model_dir(cfg, str(tmp_path), seed, dtype=torch.float32 if seed % 2 else torch.bfloat16)
    reqs = cases.requests_for(cfg["vocab_size"], lens, seed + 10)
    c, w = plain.read_model_dir(str(tmp_path), torch.float32)
    ref = {rid: plain.forward(c, w, toks) for rid, toks in reqs.items()}
    mixed_steps, peak = cases.mixed(reqs, live=4, seed=seed)
    pages = peak // page
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        eng = make_engine(str(tmp_path), dtype, page, pages, max_num_seqs=4)
        for label, steps in (("whole", cases.whole(reqs)), ("last32", cases.last_one_by_one(reqs)),
                             ("portions", cases.portions(reqs)), ("mixed", mixed_steps)):
            rows = run_steps(eng, steps)
            eng.cache.check()
            assert eng.cache.num_free == pages
            worst = max(rel_err(torch.stack([rows[(rid, i)] for i in range(len(toks))]), ref[rid])
                        for rid, toks in reqs.items())
            assert worst <= tol, (cfg, page, lens, dtype, label, worst)
