"""Parts a layer is put together from; registered by kind."""
from ..registry import register_part
from .base import (FeedForward, KvCacheSpec, Mixer, Norm, Part, PositionEncoding, StateSpec,
                   TensorDecl)
from .linear import Linear
from .norm import RmsNorm
from .rope import RopeNeox
from .mlp import SwiGluMlp
from .attention import GqaAttention
from .block import PreNormBlock

register_part("norm", "rmsnorm", RmsNorm)
register_part("position", "rope_neox", RopeNeox)
register_part("feed_forward", "swiglu", SwiGluMlp)
register_part("mixer", "gqa_attention", GqaAttention)
register_part("block", "prenorm", PreNormBlock)

__all__ = ["FeedForward", "KvCacheSpec", "Mixer", "Norm", "Part", "PositionEncoding", "StateSpec",
           "TensorDecl", "Linear", "RmsNorm", "RopeNeox", "SwiGluMlp", "GqaAttention", "PreNormBlock"]
