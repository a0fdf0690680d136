"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

    python -m infero_b200.tools.random_model --config CONFIG.json --out DIR [--seed 0]
        [--dtype bfloat16|float32] [--std 0.02] [--norm-std 0.0]

The architecture is the one CONFIG.json names; matrices, embeddings and biases are
N(0, std), norm weights 1 + N(0, norm-std).  Every tensor's values depend on the seed and the
tensor's name only.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="random_model", description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", required=True, help="a config.json of a registered architecture")
    ap.add_argument("--out", required=True, help="folder to write")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--std", type=float, default=0.02)
    ap.add_argument("--norm-std", type=float, default=0.0)
    args = ap.parse_args(argv)
    from infero_b200.loading import write_random_model_dir
    with open(args.config, "r", encoding="utf-8") as f:
        cfg = json.load(f)
    write_random_model_dir(args.out, cfg, seed=args.seed, dtype=args.dtype, std=args.std, norm_std=args.norm_std)
    print(f"wrote {args.out}/config.json and {args.out}/model.safetensors (seed {args.seed}, {args.dtype})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
