"""Architecture-neutral description of a decoder: what the parts are, layer by layer.

An architecture's own configuration (for instance ``Qwen2Config``) is read from its
``config.json`` keys and then lowered to a ``ModelSpec``.  Everything below the
architecture module works from the ``ModelSpec`` alone: parts are chosen by the ``kind``
string of their spec, sizes and constants travel inside the spec, and no part knows
which model it sits in.

The reference keeps one flat ``Config`` for every architecture
(crates/model/src/config.rs:41-110) and reads the block kind off the tensors that are
present (crates/model/src/weights.rs:810).  Here the block kind is explicit data.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


def _name_map(given, defaults) -> dict:
    known = dict(defaults)
    out = dict(known)
    for k, v in given:
        if k not in known and k not in ("qkv", "gate_up"):
            raise ValueError(f"unknown tensor role '{k}' (known: {sorted(known)})")
        out[k] = v
    return out


# Leaf names (under the block's prefix) of the tensors the built-in parts bind, as the Hugging Face
# checkpoints of the Llama / Qwen2 family store them (crates/model/src/weights.rs:3165-3205,
# :2970-3004).  An architecture that stores the same arithmetic under other names passes its own in
# ``names``; "qkv" (one [q; k; v] stacked tensor) or "gate_up" (one [gate; up] stacked tensor) may
# stand for the separate ones.
ATTENTION_NAMES = (("q", "self_attn.q_proj"), ("k", "self_attn.k_proj"), ("v", "self_attn.v_proj"),
                   ("o", "self_attn.o_proj"))
SWIGLU_NAMES = (("gate", "mlp.gate_proj"), ("up", "mlp.up_proj"), ("down", "mlp.down_proj"))


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding applied to queries and keys inside a mixer.

    kind "rope_neox": pairs (i, i + rotary_dim/2), angle = pos * theta^(-2i/rotary_dim)
    (crates/kernels/src/cu/ops.cu:488-523, crates/kernels/src/cpu/mod.rs:275-314).
    """
    kind: str
    theta: float
    rotary_dim: int


@dataclass(frozen=True)
class NormSpec:
    """kind "rmsnorm": x * rsqrt(mean(x^2) + eps) * w (crates/kernels/src/cu/ops.cu:44-62)."""
    kind: str
    dim: int
    eps: float


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of one block.

    kind "gqa_attention": grouped-query attention over the paged cache.  ``window`` is
    None for all keys, or W so that key j is visible from query p iff j <= p and
    p - j < W.
    """
    kind: str
    hidden: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    scale: float = 0.0
    window: Optional[int] = None
    position: Optional[PositionSpec] = None
    # free-form extras for mixers defined outside the framework
    extra: Tuple[Tuple[str, object], ...] = ()
    # role -> leaf name under the block's prefix (see ATTENTION_NAMES); roles not given keep the default
    names: Tuple[Tuple[str, str], ...] = ()

    def get(self, key, default=None):
        for k, v in self.extra:
            if k == key:
                return v
        return default

    def tensor_names(self) -> dict:
        return _name_map(self.names, ATTENTION_NAMES)


@dataclass(frozen=True)
class FeedForwardSpec:
    """kind "swiglu": down(silu(gate(x)) * up(x)) (crates/model/src/lib.rs:7391-7451)."""
    kind: str
    hidden: int
    intermediate: int
    extra: Tuple[Tuple[str, object], ...] = ()
    names: Tuple[Tuple[str, str], ...] = ()          # role -> leaf name (see SWIGLU_NAMES)

    def tensor_names(self) -> dict:
        return _name_map(self.names, SWIGLU_NAMES)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its parts and the tensor-name prefix its weights live under.

    kind "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)).
    """
    kind: str
    prefix: str
    mixer: MixerSpec
    ffn: FeedForwardSpec
    mixer_norm: NormSpec
    ffn_norm: NormSpec
    # leaf names of the two norm weights under the prefix
    mixer_norm_name: str = "input_layernorm.weight"
    ffn_norm_name: str = "post_attention_layernorm.weight"


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a block.

    ``block`` indexes ``ModelSpec.blocks`` (a block may be named more than once).
    ``cache`` is the cache slot this execution reads; ``write_cache`` says whether it
    appends this step's keys and values there (False lets a layer read the cache another
    execution filled).
    """
    block: int
    cache: int
    write_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    max_positions: int = 4096
    eos_token_ids: Tuple[int, ...] = ()
    embed_scale: float = 1.0
    logit_scale: float = 1.0

    def num_cache_slots(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)
