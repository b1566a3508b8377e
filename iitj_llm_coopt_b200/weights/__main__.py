"""`python -m iitj_llm_coopt_b200.weights --config config.json --out DIR --seed 3` writes a model folder
(config.json, model.safetensors) with seeded random weights for the given configuration."""
import argparse
import json
import sys

import torch

from .random_init import write_model_dir


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m iitj_llm_coopt_b200.weights", description=__doc__)
    ap.add_argument("--config", required=True, help="a config.json of a registered architecture")
    ap.add_argument("--out", required=True, help="folder to write")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--std", type=float, default=0.02, help="standard deviation of matrices and tables")
    args = ap.parse_args(argv)
    with open(args.config, encoding="utf-8") as f:
        raw = json.load(f)
    write_model_dir(raw, args.out, args.seed, dtype=getattr(torch, args.dtype), std=args.std)
    print(f"wrote {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
