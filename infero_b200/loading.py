"""From a model folder (or a configuration and a seed) to a bound model on the device."""
from __future__ import annotations

from typing import Any, Dict, Tuple

import torch

from .models.decoder import DecoderModel
from .registry import load_config, resolve_architecture
from .weights import load_tensors, random_tensors, write_random_model


def _storage_dtype(name: str) -> torch.dtype:
    return {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
            "fp32": torch.float32, "float16": torch.float16}[name]


def load_model(model_dir: str, dtype: str = "bfloat16", device="cuda:0") -> Tuple[DecoderModel, Any]:
    """Read config.json, pick the model by its architecture name, bind model.safetensors."""
    arch, cfg, spec = load_config(model_dir)
    model = DecoderModel(spec)
    tensors = load_tensors(model_dir, model.declare(), dtype, device)
    model.bind(tensors)
    return model, cfg


def random_model(config: Dict[str, Any], seed: int, dtype: str = "bfloat16", device="cuda:0",
                 std: float = 0.02, norm_std: float = 0.0, generate_on_device: bool = False
                 ) -> Tuple[DecoderModel, Any]:
    """A model with random weights made in memory (no folder).  ``generate_on_device`` draws
    the numbers on the GPU (for sizes where the host would take minutes); the values then
    differ from those of a written folder with the same seed."""
    arch = resolve_architecture(config)
    cfg = arch.read_config(config)
    spec = arch.to_spec(cfg)
    model = DecoderModel(spec)
    store = torch.float32 if dtype in ("float32", "fp32") else torch.bfloat16
    decls = model.declare()
    if generate_on_device:
        tensors = random_tensors(decls, seed, store, std, norm_std, device=device)
    else:
        tensors = {k: v.to(device) for k, v in random_tensors(decls, seed, store, std, norm_std).items()}
    model.bind(tensors)
    return model, cfg


def write_random_model_dir(model_dir: str, config: Dict[str, Any], seed: int, dtype: str = "bfloat16",
                           std: float = 0.02, norm_std: float = 0.0) -> None:
    """Random-weights mode: write ``config.json`` and ``model.safetensors`` for ``config``."""
    arch = resolve_architecture(config)
    cfg = arch.read_config(config)
    spec = arch.to_spec(cfg)
    model = DecoderModel(spec)
    cj = cfg.to_json_dict() if hasattr(cfg, "to_json_dict") else dict(config)
    cj["torch_dtype"] = "float32" if _storage_dtype(dtype) == torch.float32 else "bfloat16"
    write_random_model(model_dir, cj, model.declare(), seed, _storage_dtype(dtype), std, norm_std)
