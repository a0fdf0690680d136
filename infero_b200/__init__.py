"""infero_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token: typed configuration and an
architecture registry, safetensors weights, layers composed from parts, a paged cache
manager, one step function for mixed batches, a continuous-batching scheduler, sampling,
and hand-written CUDA kernels.
"""
from . import registry  # noqa: F401
from .config import EngineConfig, Qwen2Config
from .registry import (load_config, register_architecture, register_part, resolve_architecture)

__version__ = "0.1.0"
__all__ = ["EngineConfig", "Qwen2Config", "load_config", "register_architecture", "register_part",
           "resolve_architecture"]
