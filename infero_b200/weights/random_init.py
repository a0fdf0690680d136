"""Random-weights mode: tensors from a seed, and a model folder written from them.

Each tensor has its own generator seeded from (seed, tensor name), so a tensor's values do
not depend on which other tensors exist or in which order they are made.  Matrices,
embeddings and biases are N(0, std); norm weights are 1 (+ N(0, norm_std) when asked).
The reference has no such loader mode; its tests assemble models from synthetic device
tensors (crates/model/src/lib.rs:2500-2522).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, List

import torch

from ..parts.base import TensorDecl
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(decl: TensorDecl, seed: int, dtype: torch.dtype, std: float = 0.02,
                  norm_std: float = 0.0, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, decl.name))
    if decl.init == "ones":
        t = torch.ones(decl.shape, dtype=torch.float32, device=device)
        if norm_std > 0:
            t += torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device) * norm_std
    else:
        t = torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device) * std
    return t.to(dtype)


def random_tensors(decls: List[TensorDecl], seed: int, dtype: torch.dtype, std: float = 0.02,
                   norm_std: float = 0.0, device="cpu") -> Dict[str, torch.Tensor]:
    return {d.name: random_tensor(d, seed, dtype, std, norm_std, device) for d in decls}


def write_random_model(model_dir: str, config_json: dict, decls: List[TensorDecl], seed: int,
                       dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                       norm_std: float = 0.0) -> None:
    """Write ``config.json`` and ``model.safetensors`` for a randomly initialised model."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_json, f, indent=1)
    by_name = {d.name: d for d in decls}
    write_safetensors(
        os.path.join(model_dir, "model.safetensors"),
        [(d.name, dtype, tuple(d.shape)) for d in decls],
        lambda name: random_tensor(by_name[name], seed, dtype, std, norm_std),
        metadata={"format": "pt", "seed": str(seed)})
