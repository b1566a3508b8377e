"""The replay program's protocol, on the CPU with the plain-torch kernel double: what it writes and prints for
steps with nothing wanted, with no entries, with a request left out of a step and taken up later, and with ends of
requests it does not hold; the logits it writes against the plain implementation."""
import io
import json
import os

import numpy as np
import torch

import plain_llama as plain
from configs import CONFIGS
from iitj_llm_coopt_b200 import replay
from torch_kernels import TorchKernels


def test_replay_protocol(model_dirs, tmp_path):
    cfg, seed, page = CONFIGS["A"]
    vocab = cfg["vocab_size"]
    a = [(7 * i + 3) % vocab for i in range(40)]
    b = [(11 * i + 5) % vocab for i in range(9)]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": []}], "end": []},                       # nothing wanted
        {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": [1]}], "end": ["nobody"]},               # a is left out
        {"step": 2, "entries": [], "end": []},                                                                # nothing to do
        {"step": 3, "entries": [{"id": "a", "tokens": a[17:39], "want": [0, 21]}, {"id": "b", "tokens": b[2:3], "want": [0]}],
         "end": []},
        {"step": 7, "entries": [{"id": "b", "tokens": b[3:], "want": [5]}, {"id": "a", "tokens": a[39:], "want": [0]}],
         "end": ["a", "b"]},
        {"step": 8, "entries": [{"id": "a", "tokens": a[:3], "want": [2]}]},                                  # the id is used anew
    ]
    out_dir = tmp_path / "out"
    args = replay.parse_args(["--model", model_dirs["A"], "--dtype", "float32", "--out", str(out_dir), "--max-tokens", "128",
                              "--page-size", str(page), "--device", "cpu"])
    printed = io.StringIO()
    assert replay.run(args, [json.dumps(s) for s in steps] + ["", "  "], out=printed, kernels=TorchKernels()) == 0
    assert printed.getvalue().split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    assert sorted(os.listdir(out_dir)) == ["1.f32", "3.f32", "7.f32", "8.f32"]          # steps 0 and 2 wanted nothing
    c, w = plain.read_model_dir(model_dirs["A"], torch.float32)
    ra, rb = plain.forward(c, w, a), plain.forward(c, w, b)
    want = {1: [rb[1]], 3: [ra[17], ra[38], rb[2]], 7: [rb[8], ra[39]], 8: [ra[2]]}
    for step, rows in want.items():
        got = np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(len(rows), vocab)
        ref = torch.stack(rows).numpy()
        assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()
