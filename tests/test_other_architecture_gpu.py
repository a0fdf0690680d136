"""What another architecture needs from the framework, shown from outside the package.

Two things no file of the package is edited for: (1) an architecture whose checkpoint stores the
built-in arithmetic under other tensor names, q/k/v and gate/up as single stacked tensors among them;
(2) a mixer whose cached values are wider than its keys.  Both are registered here, built from a
config.json by their architecture name and stepped by the same runner, cache and step function.
Neither is a model of anyone's: the names and sizes are made up.
"""
import json
import math
import os
import tempfile

import numpy as np
import pytest
import torch

import plain_qwen2 as P
import replay_util as R
from engine_fixtures import TOL, make_requests, make_runner, model_dir
from tiny_configs import CONFIGS

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---- (1) the built-in parts under other tensor names ------------------------------------------------------
def _register_renamed():
    from infero_b200.config.spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                         ScheduleEntry)
    from infero_b200.registry import register_architecture

    def to_spec(c):
        d, D = c["width"], c["head"]
        norm = NormSpec("rmsnorm", d, c["eps"])
        blocks = []
        for i in range(c["depth"]):
            mixer = MixerSpec("gqa_attention", d, c["heads"], c["kv_heads"], D, qkv_bias=True, scale=1 / math.sqrt(D),
                              window=c["window"] if i >= 1 else None, position=PositionSpec("rope_neox", c["theta"], D),
                              names=(("qkv", "attn.wqkv"), ("o", "attn.wo")))
            ffn = FeedForwardSpec("swiglu", d, c["inner"], names=(("gate_up", "ffn.w13"), ("down", "ffn.w2")))
            blocks.append(BlockSpec("prenorm", f"decoder.h.{i}", mixer, ffn, norm, norm,
                                    mixer_norm_name="ln1.scale", ffn_norm_name="ln2.scale"))
        return ModelSpec("ToyRenamedForCausalLM", c["vocab"], d, tuple(blocks),
                         tuple(ScheduleEntry(i, i) for i in range(len(blocks))), norm, False,
                         embed_name="tok.weight", final_norm_name="ln_f.scale", head_name="out.weight",
                         max_positions=c["max_pos"])

    register_architecture("ToyRenamedForCausalLM", dict, to_spec)


def _renamed_folder(src: str, dst: str) -> None:
    """The tensors of a Qwen2 folder under the made-up names, q/k/v and gate/up stacked as stored tensors."""
    from safetensors.torch import load_file, save_file
    q = CONFIGS["D"]
    w = load_file(os.path.join(src, "model.safetensors"))
    out = {"tok.weight": w["model.embed_tokens.weight"], "ln_f.scale": w["model.norm.weight"], "out.weight": w["lm_head.weight"]}
    for i in range(q["num_hidden_layers"]):
        a, b = f"model.layers.{i}.", f"decoder.h.{i}."
        out[b + "attn.wqkv.weight"] = torch.cat([w[a + f"self_attn.{p}_proj.weight"] for p in "qkv"])
        out[b + "attn.wqkv.bias"] = torch.cat([w[a + f"self_attn.{p}_proj.bias"] for p in "qkv"])
        out[b + "attn.wo.weight"] = w[a + "self_attn.o_proj.weight"]
        out[b + "ffn.w13.weight"] = torch.cat([w[a + "mlp.gate_proj.weight"], w[a + "mlp.up_proj.weight"]])
        out[b + "ffn.w2.weight"] = w[a + "mlp.down_proj.weight"]
        out[b + "ln1.scale"] = w[a + "input_layernorm.weight"]
        out[b + "ln2.scale"] = w[a + "post_attention_layernorm.weight"]
    os.makedirs(dst, exist_ok=True)
    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(dst, "model.safetensors"))
    cfg = {"architectures": ["ToyRenamedForCausalLM"], "width": q["hidden_size"], "inner": q["intermediate_size"],
           "vocab": q["vocab_size"], "depth": q["num_hidden_layers"], "heads": q["num_attention_heads"],
           "kv_heads": q["num_key_value_heads"], "head": q["head_dim"], "eps": q["rms_norm_eps"],
           "theta": q["rope_theta"], "window": q["sliding_window"], "max_pos": q["max_position_embeddings"]}
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(cfg, f)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_architecture_with_other_tensor_names_reuses_the_parts(dtype):
    from infero_b200.loading import load_model
    from infero_b200.parts import native_block
    from infero_b200.weights import WeightsError
    _register_renamed()
    src = model_dir("D")
    with tempfile.TemporaryDirectory(prefix="infero_b200_renamed_") as dst:
        _renamed_folder(src, dst)
        model, _ = load_model(dst, dtype, DEV)
        names = {d.name for d in model.declare()}
        assert "decoder.h.1.attn.wqkv.bias" in names and "decoder.h.2.ffn.w13.weight" in names and "out.weight" in names
        assert not any("self_attn" in n or "mlp." in n or n.startswith("model.") for n in names)
        reqs = make_requests("D", [150, 40, 97], seed=3)
        steps = R.steps_mixed(reqs, seed=1, max_live=3)
        n = R.max_live_tokens(steps, reqs)
        calls = native_block.CALLS[0]
        got = R.replay_inprocess(make_runner(dst, dtype, n), steps)
        if dtype == "bfloat16":
            assert native_block.CALLS[0] > calls, "the renamed architecture did not reach the native launcher"
        same = R.replay_inprocess(make_runner(src, dtype, n), steps)
        assert got.keys() == same.keys()
        for key in got:                                 # the same arithmetic on the same numbers
            assert np.array_equal(got[key], same[key]), key
        # a Qwen2 folder does not load as this architecture, and the one error says so in its names
        with pytest.raises(WeightsError) as e:
            from infero_b200.weights import load_tensors
            load_tensors(src, model.declare(), dtype, "cpu")
        assert "decoder.h.0.attn.wqkv.weight" in e.value.missing
        assert "model.layers.0.self_attn.q_proj.weight" in e.value.unexpected


# ---- (2) a mixer whose values are wider than its keys ----------------------------------------------------------
WIDE = {"architectures": ["ToyWideValueForCausalLM"], "width": 48, "inner": 100, "vocab": 173, "eps": 1e-5,
        "heads": 3, "key": 16, "value": 40, "depth": 2}


def _register_wide_value():
    from infero_b200.config.spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, ScheduleEntry)
    from infero_b200.parts.base import KvCacheSpec, Mixer, TensorDecl
    from infero_b200.registry import register_architecture, register_part

    class WideValueAttention(Mixer):
        """Causal attention without positions: keys of width ``key``, values of width ``value``, one kv
        head per head.  It keeps both in the paged cache the framework gives it (two arrays of
        different widths) and finds them through the block table, with torch for its arithmetic."""

        def __init__(self, spec, prefix):
            self.spec, self.prefix = spec, prefix
            self.H, self.Dk, self.Dv = spec.num_heads, spec.get("key"), spec.get("value")

        def _names(self):
            H, Dk, Dv, d = self.H, self.Dk, self.Dv, self.spec.hidden
            return {"wq": (H * Dk, d), "wk": (H * Dk, d), "wv": (H * Dv, d), "wo": (d, H * Dv)}

        def declare(self):
            return [TensorDecl(f"{self.prefix}.mix.{n}", shape) for n, shape in self._names().items()]

        def bind(self, tensors):
            self.w = {n: tensors[f"{self.prefix}.mix.{n}"].float() for n in self._names()}

        def cache_spec(self):
            return KvCacheSpec(self.H, self.Dk, None, v_head_dim=self.Dv)

        def forward(self, ctx, h, slot):
            H, Dk, Dv = self.H, self.Dk, self.Dv
            kv = ctx.kv_cache(slot.cache)
            assert kv.k.shape[1:] == (H, kv.page_size, Dk) and kv.v.shape[1:] == (H, kv.page_size, Dv)
            table = ctx.block_table(kv.group)
            x = h.float()
            q = (x @ self.w["wq"].T).view(-1, H, Dk)
            k = (x @ self.w["wk"].T).view(-1, H, Dk)
            v = (x @ self.w["wv"].T).view(-1, H, Dv)
            pos, ent = ctx.positions.long(), ctx.tok_entry.long()
            page = table[ent, pos // kv.page_size].long()
            kv.k[page, :, pos % kv.page_size] = k.to(kv.k.dtype)
            kv.v[page, :, pos % kv.page_size] = v.to(kv.v.dtype)
            out = torch.empty((x.shape[0], H * Dv), dtype=torch.float32, device=x.device)
            for t in range(x.shape[0]):
                js = torch.arange(int(pos[t]) + 1, device=x.device)
                pages = table[ent[t], js // kv.page_size].long()
                keys = kv.k[pages, :, js % kv.page_size].float()          # [n, H, Dk]
                vals = kv.v[pages, :, js % kv.page_size].float()
                s = torch.einsum("hd,nhd->hn", q[t], keys) / math.sqrt(Dk)
                out[t] = torch.einsum("hn,nhd->hd", torch.softmax(s, dim=-1), vals).reshape(-1)
            return (out @ self.w["wo"].T).to(h.dtype)

    def to_spec(c):
        d = c["width"]
        norm = NormSpec("rmsnorm", d, c["eps"])
        blocks = [BlockSpec("prenorm", f"model.layers.{i}",
                            MixerSpec("wide_value_attention", d, c["heads"], extra=(("key", c["key"]), ("value", c["value"]))),
                            FeedForwardSpec("swiglu", d, c["inner"]), norm, norm) for i in range(c["depth"])]
        return ModelSpec("ToyWideValueForCausalLM", c["vocab"], d, tuple(blocks),
                         tuple(ScheduleEntry(i, i) for i in range(len(blocks))), norm, True)

    register_part("mixer", "wide_value_attention", WideValueAttention)
    register_architecture("ToyWideValueForCausalLM", dict, to_spec)


def _wide_plain(w, toks):
    c = WIDE
    H, Dk, Dv = c["heads"], c["key"], c["value"]
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    T = len(toks)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for i in range(c["depth"]):
        p = f"model.layers.{i}."
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
        q = (h @ w[p + "mix.wq"].T).view(T, H, Dk)
        k = (h @ w[p + "mix.wk"].T).view(T, H, Dk)
        v = (h @ w[p + "mix.wv"].T).view(T, H, Dv)
        s = torch.einsum("thd,nhd->htn", q, k) / math.sqrt(Dk)
        s = s.masked_fill(~causal, float("-inf"))
        a = torch.einsum("htn,nhd->thd", torch.softmax(s, dim=-1), v).reshape(T, H * Dv)
        x = x + a @ w[p + "mix.wo"].T
        h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
        x = x + P.swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.rms_norm(x, w["model.norm.weight"], c["eps"]) @ w["model.embed_tokens.weight"].T


def test_a_mixer_with_values_wider_than_keys_plugs_in():
    from infero_b200.loading import load_model, write_random_model_dir
    _register_wide_value()
    with tempfile.TemporaryDirectory(prefix="infero_b200_wide_value_") as tmp:
        write_random_model_dir(tmp, WIDE, seed=9, dtype="float32", std=0.1, norm_std=0.1)
        model, _ = load_model(tmp, "float32", DEV)
        _, w = P.read_model(tmp, torch.float64)
        spec = model.kv_specs[0]
        assert (spec.head_dim, spec.value_dim) == (16, 40)
        g = torch.Generator().manual_seed(2)
        reqs = {f"r{i}": [int(t) for t in torch.randint(0, WIDE["vocab"], (n,), generator=g)]
                for i, n in enumerate([45, 20, 33, 50])}
        plain = {r: _wide_plain(w, t).numpy() for r, t in reqs.items()}
        steps = R.steps_mixed(reqs, seed=4, max_live=3)
        runner = make_runner(tmp, "float32", R.max_live_tokens(steps, reqs))
        k, v = runner.storage.k_arrays[0], runner.storage.v_arrays[0]
        assert k.shape[-1] == 16 and v.shape[-1] == 40 and k.shape[:-1] == v.shape[:-1]
        got = R.replay_inprocess(runner, steps)
        err, where = R.compare(got, plain)
        assert err <= TOL["float32"], f"relative error {err:.3e} at {where}"
        assert runner.manager.pages_reused > 0
