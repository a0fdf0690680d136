"""Shared builders for the GPU tests: model folders, runners, plain logits."""
from __future__ import annotations

import functools
import os
import random
import tempfile
from typing import Dict, List

import numpy as np
import torch

import plain_qwen2
from tiny_configs import CONFIGS, NORM_STD, STORE

_TMP = tempfile.mkdtemp(prefix="infero_b200_tests_")

# Tolerances: largest |engine - plain| over a row, relative to the largest |logit| of the
# request.  float32 is the engine's 32-bit path against the 64-bit plain forward (observed
# errors are a few 1e-6).  bfloat16 rounds every activation handed to a product and every
# cached key and value to 8 mantissa bits (2^-9 = 2e-3 per rounding), and a few dozen of
# those roundings feed each logit.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


@functools.lru_cache(maxsize=None)
def model_dir(name: str, store: str = None, seed: int = 1234, qk_gain: float = 1.0) -> str:
    """A random model folder (made once per process, in a temporary folder).  ``store``: the dtype
    the tensors are written in (by default A, B, C in float32, D and E in bfloat16)."""
    from infero_b200.loading import write_random_model_dir
    store = store or STORE[name]
    d = os.path.join(_TMP, f"tiny_{name}_{store}_{seed}_{qk_gain}")
    write_random_model_dir(d, CONFIGS[name], seed=seed, dtype=store, std=0.02 if qk_gain == 1.0 else 0.05,
                           norm_std=NORM_STD[name])
    if qk_gain != 1.0:
        # sharpen attention: random 0.02 weights give almost flat softmax, which hides wrong
        # keys; scale the q and k projections so that scores differ by several units
        from safetensors.torch import load_file, save_file
        p = os.path.join(d, "model.safetensors")
        w = load_file(p)
        for k in list(w):
            if "q_proj" in k or "k_proj" in k:
                w[k] = (w[k].float() * qk_gain).to(w[k].dtype)
        save_file(w, p, metadata={"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def plain_model(mdir: str):
    return plain_qwen2.read_model(mdir, torch.float64)


def plain_logits(mdir: str, reqs: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    cfg, w = plain_model(mdir)
    return {rid: plain_qwen2.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def make_requests(name: str, lengths, seed: int = 0) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    V = CONFIGS[name]["vocab_size"]
    return {f"r{i}": [rng.randrange(V) for _ in range(n)] for i, n in enumerate(lengths)}


def make_runner(mdir: str, dtype: str, max_tokens: int, page_size: int = 16, max_seqs: int = 8,
                cuda_graphs: bool = False, **kw):
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner
    from infero_b200.loading import load_model
    model, _ = load_model(mdir, dtype, "cuda:0")
    pages = -(-max_tokens // page_size)
    cfg = EngineConfig(dtype=dtype, page_size=page_size, num_pages=pages, max_seqs=max_seqs,
                       ctx=pages * page_size, max_batch_tokens=max(64, pages * page_size),
                       max_logit_rows=max(64, pages * page_size), cuda_graphs=cuda_graphs, **kw)
    return ModelRunner(model, cfg)
