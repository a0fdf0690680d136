"""Typed configuration of the Qwen2 dense decoder, read from its own config.json keys.

Keys and defaults follow the reference's HF reader (crates/model/src/config.rs:492-719):
``hidden_size``, ``num_attention_heads``, ``num_hidden_layers``, ``intermediate_size`` and
``vocab_size`` are required; ``num_key_value_heads`` defaults to the head count and
``head_dim`` to hidden/heads (:519-530); ``rms_norm_eps`` defaults to 1e-5 (:642),
``rope_theta`` to 10000 and may sit under ``rope_parameters`` (:556-560),
``max_position_embeddings`` to 4096 (:641), ``tie_word_embeddings`` to false (:654-657);
a nested ``text_config`` is preferred when present (:499-503).  The reference has no
sliding window; ``use_sliding_window`` / ``sliding_window`` / ``max_window_layers`` (and
an explicit ``layer_types`` list) are read here as the architecture's config.json names
them: layer i uses the window iff use_sliding_window and i >= max_window_layers.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec, ScheduleEntry)

# Where a Qwen2 checkpoint keeps a layer's tensors, under ``model.layers.<i>``
# (crates/model/src/weights.rs:3165-3205, :2970-3004, :3349-3355).
ATTENTION_TENSORS = (("q", "self_attn.q_proj"), ("k", "self_attn.k_proj"), ("v", "self_attn.v_proj"),
                     ("o", "self_attn.o_proj"))
MLP_TENSORS = (("gate", "mlp.gate_proj"), ("up", "mlp.up_proj"), ("down", "mlp.down_proj"))


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model."""


def _require(d: Dict[str, Any], key: str, typ=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if typ is int and (isinstance(v, bool) or not isinstance(v, int)):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if typ is int and v <= 0:
        raise ConfigError(f"config.json: '{key}' must be positive, got {v}")
    return v


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    layer_types: Optional[Tuple[str, ...]] = None
    hidden_act: str = "silu"
    attention_bias: bool = True
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    model_type: str = "qwen2"
    architectures: Tuple[str, ...] = ("Qwen2ForCausalLM",)

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen2Config":
        d = dict(raw)
        if isinstance(d.get("text_config"), dict):
            outer = d
            d = dict(d["text_config"])
            for k in ("architectures", "tie_word_embeddings", "torch_dtype", "eos_token_id"):
                if k not in d and k in outer:
                    d[k] = outer[k]
        hidden = _require(d, "hidden_size")
        heads = _require(d, "num_attention_heads")
        layers = _require(d, "num_hidden_layers")
        inter = _require(d, "intermediate_size")
        vocab = _require(d, "vocab_size")
        kv_heads = d.get("num_key_value_heads")
        if kv_heads is None:
            kv_heads = heads
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not divisible by num_attention_heads "
                    f"{heads} and no head_dim is given")
            head_dim = hidden // heads
        rope_theta = d.get("rope_theta")
        if rope_theta is None and isinstance(d.get("rope_parameters"), dict):
            rope_theta = d["rope_parameters"].get("rope_theta")
        if rope_theta is None:
            rope_theta = 10000.0
        scaling = d.get("rope_scaling")
        if scaling is None and isinstance(d.get("rope_parameters"), dict):
            rp = d["rope_parameters"]
            if rp.get("rope_type", "default") not in ("default", None):
                scaling = rp
        if scaling not in (None, {}):
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling {scaling!r} is not supported by Qwen2 here")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(e) for e in eos)
        lt = d.get("layer_types")
        cfg = cls(
            vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
            num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=int(kv_heads), head_dim=int(head_dim),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            rope_theta=float(rope_theta),
            partial_rotary_factor=float(d.get("partial_rotary_factor", 1.0)),
            max_position_embeddings=int(d.get("max_position_embeddings", 4096)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=(None if d.get("sliding_window") is None else int(d["sliding_window"])),
            max_window_layers=int(d.get("max_window_layers", 0) or 0),
            layer_types=(None if lt is None else tuple(str(t) for t in lt)),
            hidden_act=str(d.get("hidden_act", "silu")),
            attention_bias=bool(d.get("attention_bias", True)),
            eos_token_ids=eos_ids,
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            model_type=str(d.get("model_type", "qwen2")),
            architectures=tuple(d.get("architectures") or ("Qwen2ForCausalLM",)),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "Qwen2Config":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    # ---- checks (crates/model/src/config.rs:523-542, :574-578) --------------------
    def validate(self) -> None:
        if self.num_key_value_heads <= 0 or self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} must be a positive "
                f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim <= 0 or self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be positive and even")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (silu only)")
        if not (0.0 < self.partial_rotary_factor <= 1.0):
            raise ConfigError(f"config.json: partial_rotary_factor {self.partial_rotary_factor} out of (0, 1]")
        if self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ConfigError(f"config.json: rotary dimension {self.rotary_dim} must be positive and even")
        if self.rms_norm_eps <= 0 or not math.isfinite(self.rms_norm_eps):
            raise ConfigError(f"config.json: rms_norm_eps {self.rms_norm_eps} must be positive")
        if self.rope_theta <= 0:
            raise ConfigError(f"config.json: rope_theta {self.rope_theta} must be positive")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            raise ConfigError("config.json: use_sliding_window is true but sliding_window is missing or <= 0")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(
                    f"config.json: layer_types has {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers")
            for t in self.layer_types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"config.json: unknown layer type '{t}'")
            if "sliding_attention" in self.layer_types and not self.sliding_window:
                raise ConfigError("config.json: layer_types names sliding_attention but sliding_window is missing")
        for e in self.eos_token_ids:
            if not (0 <= e < self.vocab_size):
                raise ConfigError(f"config.json: eos_token_id {e} outside the vocabulary")

    # ---- derived (crates/model/src/config.rs:309-316, :917-925) -------------------
    @property
    def rotary_dim(self) -> int:
        return int(round(self.head_dim * self.partial_rotary_factor))

    @property
    def attn_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, i: int) -> Optional[int]:
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[i] == "sliding_attention" else None
        if self.use_sliding_window and i >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_json_dict(self) -> Dict[str, Any]:
        d = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "torch_dtype": self.torch_dtype,
        }
        if self.partial_rotary_factor != 1.0:
            d["partial_rotary_factor"] = self.partial_rotary_factor
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        return d

    # ---- lowering to parts ---------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        """Qwen2 block: pre-norm, GQA attention with q/k/v bias and NeoX rotary, SwiGLU
        (crates/metal/examples/qwen2_f16.rs:863-935; README.md:206-218)."""
        pos = PositionSpec(kind="rope_neox", theta=self.rope_theta, rotary_dim=self.rotary_dim)
        blocks: List[BlockSpec] = []
        for i in range(self.num_hidden_layers):
            prefix = f"model.layers.{i}"
            mixer = MixerSpec(
                kind="gqa_attention", hidden=self.hidden_size,
                num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim, qkv_bias=self.attention_bias, out_bias=False,
                scale=1.0 / math.sqrt(self.head_dim),   # crates/model/src/config.rs:923-925
                window=self.layer_window(i), position=pos, names=ATTENTION_TENSORS)
            ffn = FeedForwardSpec(kind="swiglu", hidden=self.hidden_size,
                                  intermediate=self.intermediate_size, names=MLP_TENSORS)
            norm = NormSpec(kind="rmsnorm", dim=self.hidden_size, eps=self.rms_norm_eps)
            blocks.append(BlockSpec(kind="prenorm", prefix=prefix, mixer=mixer, ffn=ffn,
                                    mixer_norm=norm, ffn_norm=norm,
                                    mixer_norm_name="input_layernorm.weight",
                                    ffn_norm_name="post_attention_layernorm.weight"))
        schedule = tuple(ScheduleEntry(block=i, cache=i) for i in range(self.num_hidden_layers))
        return ModelSpec(
            architecture="Qwen2ForCausalLM", vocab_size=self.vocab_size, hidden=self.hidden_size,
            blocks=tuple(blocks), schedule=schedule,
            final_norm=NormSpec(kind="rmsnorm", dim=self.hidden_size, eps=self.rms_norm_eps),
            tie_embeddings=self.tie_word_embeddings,
            embed_name="model.embed_tokens.weight", final_norm_name="model.norm.weight",
            head_name="lm_head.weight",
            max_positions=self.max_position_embeddings,
            eos_token_ids=self.eos_token_ids)
