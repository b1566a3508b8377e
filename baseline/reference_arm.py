"""The benchmark's reference arm: the unmodified engine of mohsinmubarak/iitj-llm-coopt, timed on the
same metric and configuration as this repository's own arm.

The reference is a folder of scripts (no setup.py, no pyproject.toml), so it cannot be pip-installed; a
plain copy of its tree under `baseline/_ref` on `sys.path` is what `import engine.engine` needs.  Nothing of
this repository's package is imported here: the model folder is written with torch and safetensors alone
(random weights N(0, 0.02), norm gains 1 + U(-0.1, 0.1), bfloat16, from a seed), and everything timed is the
reference's own code:

  * `Engine(target=folder, policy=StaticPolicy(gamma=0, ...), kv_gb=..., cuda_graphs=True)` (engine/engine.py:158),
    which loads the folder with `Llama.from_pretrained` (engine/model.py:134), allocates the paged cache
    (engine/model.py:148) and captures its decode graphs (engine/cuda_graphs.py:39);
  * device-timed decode: per step `Engine._run` (engine/engine.py:312: a captured graph for decode-shaped
    batches, else `build_batch` + `forward`) and the whole-step greedy shortcut `logits.argmax(-1).tolist()`
    (engine/engine.py:421-423), the sampled ids fed back as the next step's tokens; contexts are "already in
    the cache": pages reserved with `BlockManager.ensure`, keys and values random;
  * prefill: `build_batch` + `Llama.forward` of one prompt (engine/batch.py:23, engine/model.py:178);
  * end to end: `Sequence`s appended to `scheduler.waiting` and `Engine.step()` in a loop, the reference's
    in-process usage (tests/elastic_check.py:24-38), host token ids in, host token ids out through `on_output`.

If the reference cannot be imported or run here, `run()` returns {"impl": "reference", "unavailable": why}.
"""
from __future__ import annotations

import contextlib
import json
import os
import shutil
import statistics
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_TREE = os.path.join(HERE, "_ref")


def write_model_dir(cfg: dict, path: str, seed: int) -> None:
    """config.json and sharded safetensors with the checkpoint names the reference reads
    (engine/model.py:104-117); weights are drawn on the GPU and written a few layers per file."""
    import torch
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    g = torch.Generator(device="cuda").manual_seed(seed)
    h, inter, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def matrix(rows, cols):
        return (torch.randn((rows, cols), generator=g, device="cuda") * 0.02).to(torch.bfloat16).cpu()

    def gain(n):
        return (1.0 + (torch.rand((n,), generator=g, device="cuda") * 0.2 - 0.1)).to(torch.bfloat16).cpu()

    shard, count = {}, 0

    def flush():
        nonlocal shard, count
        if shard:
            save_file(shard, os.path.join(path, f"model-{count:05d}.safetensors"))
            shard, count = {}, count + 1

    shard["model.embed_tokens.weight"] = matrix(V, h)
    flush()
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shard[p + "input_layernorm.weight"] = gain(h)
        shard[p + "post_attention_layernorm.weight"] = gain(h)
        shard[p + "self_attn.q_proj.weight"] = matrix(H * D, h)
        shard[p + "self_attn.k_proj.weight"] = matrix(Hkv * D, h)
        shard[p + "self_attn.v_proj.weight"] = matrix(Hkv * D, h)
        shard[p + "self_attn.o_proj.weight"] = matrix(h, H * D)
        shard[p + "mlp.gate_proj.weight"] = matrix(inter, h)
        shard[p + "mlp.up_proj.weight"] = matrix(inter, h)
        shard[p + "mlp.down_proj.weight"] = matrix(h, inter)
        if i % 4 == 3:
            flush()
    shard["model.norm.weight"] = gain(h)
    if not cfg.get("tie_word_embeddings"):
        shard["lm_head.weight"] = matrix(V, h)
    flush()


def run(cfg: dict, model_name: str, full_layers: int, B: int, C: int, K: int, W: int, prefill_tokens: int,
        points: bool, e2e: bool, prefill: bool, peaks: dict, peak_source: str, clock_sampler, weight_bytes: int,
        prefill_flops: int, log=sys.stderr) -> dict:
    if not os.path.isdir(os.path.join(REF_TREE, "engine")):
        return {"impl": "reference", "unavailable": f"no copy of the reference tree under {os.path.relpath(REF_TREE)}"}
    import torch
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device is visible"}
    sys.path.insert(0, REF_TREE)
    try:
        with contextlib.redirect_stdout(log):
            from engine.batch import WorkItem, build_batch
            from engine.engine import Engine, Sequence
            from engine.policy import StaticPolicy
    except BaseException as e:          # vLLM's ops failing to load raise ImportError or OSError
        return {"impl": "reference", "unavailable": f"import of the reference engine failed: {type(e).__name__}: {str(e)[:300]}"}

    page = 16
    biggest = max(B, 64 if points else 1)
    pool_tokens = biggest * (C + max(K, 96) + W + 2 * page) + prefill_tokens + 4 * page
    kv_bytes_per_token = 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    kv_gb = pool_tokens * kv_bytes_per_token / 2**30
    folder = tempfile.mkdtemp(prefix="reference_model_")
    t_build = time.time()
    try:
        print(f"[reference arm] writing a random {model_name} folder to {folder}", file=log, flush=True)
        write_model_dir(cfg, folder, seed=2)
        torch.cuda.empty_cache()
        with contextlib.redirect_stdout(log):
            # the token budget lets the end-to-end phase prefill its B prompts in one step, as the other arm does, so
            # that all B requests decode together from the first decode step to the last
            eng = Engine(folder, None, policy=StaticPolicy(gamma=0, max_num_seqs=max(biggest, 8),
                                                           max_batched_tokens=max(8192, B * C if e2e else 0)),
                         kv_gb=kv_gb, max_model_len=C + max(K, 96) + W + 64, block_size=page, seed=0, cuda_graphs=True)
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    model, bm = eng.target, eng.bm
    for t in list(model.k_cache) + list(model.v_cache):           # contexts "already in the cache"
        t.normal_(0.0, 0.5)
    torch.cuda.synchronize()
    build_s = time.time() - t_build
    gen = torch.Generator().manual_seed(0)
    V = cfg["vocab_size"]
    next_id = [1 << 20]

    def decode_run(batch, steps, warmup):
        ids = list(range(next_id[0], next_id[0] + batch))
        next_id[0] += batch
        for sid in ids:
            bm.ensure(sid, C)
        toks = torch.randint(0, V, (batch,), generator=gen).tolist()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for it in range(warmup + steps):
            if it == warmup:
                torch.cuda.synchronize()
                start.record()
            items = [WorkItem(sid, [t], C + it) for sid, t in zip(ids, toks)]
            logits, spans = Engine._run(model, eng.target_graphs, bm, items)
            greedy = logits.argmax(-1).tolist()
            toks = [greedy[row] for row, _ in spans]
        end.record()
        torch.cuda.synchronize()
        for sid in ids:
            bm.free(sid)
        return start.elapsed_time(end) / steps

    def prefill_run(T, reps, warmup):
        times = []
        for it in range(warmup + reps):
            sid = next_id[0]
            next_id[0] += 1
            toks = torch.randint(0, V, (T,), generator=gen).tolist()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            batch, _ = build_batch([WorkItem(sid, toks, 0)], bm)
            model.forward(batch)
            end.record()
            torch.cuda.synchronize()
            bm.free(sid)
            if it >= warmup:
                times.append(start.elapsed_time(end))
        return times

    clock_sampler.start()
    with clock_sampler.busy():
        ms = decode_run(B, K, W)
    value = B / (ms / 1e3)
    kv_bytes = B * (C + W + K / 2) * kv_bytes_per_token
    achieved = (weight_bytes + kv_bytes) / (ms / 1e3) / 1e9

    pre = None
    if prefill:
        with clock_sampler.busy():
            p_ms = statistics.median(prefill_run(prefill_tokens, 5, 3))
        pre = {"value": prefill_tokens / (p_ms / 1e3), "tokens": prefill_tokens, "ms": p_ms,
               "frac": prefill_flops / (p_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), "peak": f"of {peak_source}"}
    pts = {}
    if points:
        for b in (1, 64):
            with clock_sampler.busy():
                pts[f"decode_b{b}"] = b / (decode_run(b, max(8, K // 2), W) / 1e3)

    e2e_rec = None
    if e2e:
        prompts = [torch.randint(0, V, (C,), generator=gen).tolist() for _ in range(B)]
        stamps = []

        def on_out(seq, new, fin):
            stamps.append(time.perf_counter())

        WE, KE = max(W, 24), max(K, 64)
        seqs = [Sequence(seq_id=i, tokens=list(p), max_tokens=WE + KE + 1, temperature=0.0, ignore_eos=True,
                         on_output=on_out) for i, p in enumerate(prompts)]
        eng.scheduler.waiting.extend(seqs)
        with clock_sampler.busy():
            while not all(s.finished for s in seqs):
                if not eng.step():
                    break
            torch.cuda.synchronize()
        per_step = sorted(stamps)
        t_start, t_last = per_step[B * (WE + 1) - 1], per_step[-1]
        decoded = len(per_step) - B * (WE + 1)
        width = -(-(eng.max_model_len + 1) // page)
        # what engine/cuda_graphs.py:84-103 copies per decode step: ids, positions, slots (int64), lengths, block table
        h2d = B * (8 + 8 + 8 + 4 + 4 * width)
        e2e_rec = {"value": decoded / (t_last - t_start), "unit": "tok/s", "steps": decoded // B, "warmup": WE,
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8 * B}
    clock_rec = clock_sampler.stop()

    return {
        "metric": f"decode tok/s at batch {B} ({model_name[:-13]} shape, {C}-token contexts); prefill and batch 1/64 alongside",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": {"model": model_name, "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": B, "seq_len": C, "page_size": page, "parallelism": "single-gpu",
                   "l2": f"inputs larger than L2 (a step reads {weight_bytes / 1e9:.1f} GB of weights)", "weights": "random seed 2",
                   "path": "Engine._run + argmax().tolist() per step, CUDA graphs on (the reference's stock decode path)"},
        "clocks": clock_rec,
        "e2e": e2e_rec,
        "gpu_launches": None,
        "prefill": pre,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peak_source": f"of {peak_source}"},
        "points": pts,
        "build_seconds": build_s,
    }
