"""Configuration and registry (no GPU)."""
import json
import math

import pytest

from infero_b200.config import Qwen2Config, ConfigError
from infero_b200.registry import (UnknownArchitecture, load_config, register_architecture,
                                  resolve_architecture)
from tiny_configs import TINY_A, TINY_B


def test_reads_every_size_from_its_keys():
    a, b = Qwen2Config.from_dict(TINY_A), Qwen2Config.from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 3, 1, 32)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.rms_norm_eps == 1e-6 and b.rms_norm_eps == 1e-5
    assert a.rope_theta == 1e4 and b.rope_theta == 1e6
    assert [a.layer_window(i) for i in range(2)] == [None, None]
    assert [b.layer_window(i) for i in range(3)] == [None, 48, 48]


def test_defaults_follow_the_reference():
    c = Qwen2Config.from_dict({"hidden_size": 64, "num_attention_heads": 4, "num_hidden_layers": 1,
                               "intermediate_size": 128, "vocab_size": 100})
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.max_position_embeddings == 4096
    assert not c.tie_word_embeddings and not c.use_sliding_window


def test_rope_parameters_and_text_config():
    raw = {"architectures": ["Qwen2ForCausalLM"], "tie_word_embeddings": True,
           "text_config": {"hidden_size": 32, "num_attention_heads": 2, "num_hidden_layers": 1,
                           "intermediate_size": 64, "vocab_size": 50,
                           "rope_parameters": {"rope_theta": 5e5, "rope_type": "default"}}}
    c = Qwen2Config.from_dict(raw)
    assert c.rope_theta == 5e5 and c.tie_word_embeddings and c.hidden_size == 32


def test_layer_types_override():
    raw = dict(TINY_B, layer_types=["sliding_attention", "full_attention", "sliding_attention"])
    c = Qwen2Config.from_dict(raw)
    assert [c.layer_window(i) for i in range(3)] == [48, None, 48]
    with pytest.raises(ConfigError):
        Qwen2Config.from_dict(dict(TINY_B, layer_types=["full_attention"]))


@pytest.mark.parametrize("patch,word", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"vocab_size": -5}, "vocab_size"),
    ({"eos_token_id": 99999}, "eos_token_id"),
])
def test_bad_configs_are_refused_with_the_key_named(patch, word):
    with pytest.raises(ConfigError) as e:
        Qwen2Config.from_dict(dict(TINY_A, **patch))
    assert word in str(e.value)


def test_spec_has_one_block_per_layer_with_its_own_window():
    spec = Qwen2Config.from_dict(TINY_B).to_model_spec()
    assert len(spec.blocks) == 3 and [e.block for e in spec.schedule] == [0, 1, 2]
    assert [b.mixer.window for b in spec.blocks] == [None, 48, 48]
    m = spec.blocks[0].mixer
    assert m.scale == pytest.approx(1 / math.sqrt(32)) and m.qkv_bias and not m.out_bias
    assert m.position.kind == "rope_neox" and m.position.rotary_dim == 32 and m.position.theta == 1e6
    assert spec.blocks[1].ffn.intermediate == 256 and spec.final_norm.eps == 1e-5


def test_registry_by_architecture_name(tmp_path):
    arch = resolve_architecture(TINY_A)
    assert arch.name == "Qwen2ForCausalLM"
    assert resolve_architecture({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"
    with pytest.raises(UnknownArchitecture) as e:
        resolve_architecture({"architectures": ["NopeForCausalLM"]})
    assert "Qwen2ForCausalLM" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg, spec = load_config(str(tmp_path))
    assert spec.vocab_size == 1000 and cfg.sliding_window == 48


def test_another_architecture_registers_without_touching_the_package():
    register_architecture("ToyArch", lambda raw: Qwen2Config.from_dict(dict(TINY_A, **raw.get("over", {}))),
                          lambda c: c.to_model_spec())
    arch = resolve_architecture({"architectures": ["ToyArch"], "over": {"vocab_size": 77}})
    assert arch.to_spec(arch.read_config({"over": {"vocab_size": 77}})).vocab_size == 77


def test_json_round_trip():
    c = Qwen2Config.from_dict(TINY_B)
    assert Qwen2Config.from_dict(c.to_json_dict()) == c
