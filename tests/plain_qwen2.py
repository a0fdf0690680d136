"""Plain, slow Qwen2 forward: whole sequences, no cache, one function per part.

This file rests on the reference's formulas, not on its compiled code: the reference is a
Rust workspace and no Rust toolchain exists here, so none of its model code can be built or
imported.  Each function cites the lines it restates.  It shares no code with the package
under test: it reads config.json with ``json`` and the weights with the ``safetensors``
package, and computes in the dtype it is given (float64 by default).

The sliding window is not in the reference (it has none); its rule is the architecture's:
layer i uses the window iff use_sliding_window and i >= max_window_layers, and key j is
visible from query p iff j <= p and p - j < sliding_window.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def read_model(model_dir: str, dtype=torch.float64):
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights: Dict[str, torch.Tensor] = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, fn), framework="pt") as sf:
                for k in sf.keys():
                    weights[k] = sf.get_tensor(k).to(dtype)
    return cfg, weights


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """crates/kernels/src/cu/ops.cu:44-62; crates/metal/examples/qwen2_f16.rs:797-801:
    s = 1/sqrt(mean(x^2) + eps); out = x * s * w."""
    s = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * s * w


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta: float, rotary_dim: int) -> torch.Tensor:
    """crates/metal/examples/qwen2_f16.rs:803-817; crates/kernels/src/cpu/mod.rs:275-314.
    x [T, heads, d]; pairs (i, i + rotary_dim/2); inv = theta^(-2i/rotary_dim)."""
    half = rotary_dim // 2
    i = torch.arange(half, dtype=torch.float64, device=x.device)
    inv = (theta ** (-2.0 * i / rotary_dim)).to(x.dtype)
    ang = positions.to(x.dtype)[:, None] * inv[None, :]            # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = a * c - b * s
    out[..., half:rotary_dim] = a * s + b * c
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: Optional[int]) -> torch.Tensor:
    """crates/metal/examples/qwen2_f16.rs:879-909; crates/kernels/src/cu/ops.cu:709-811.
    q [T, H, d], k/v [T, Hkv, d]; kv head = h // group; scores * scale, causal mask,
    softmax with max subtraction, weighted sum of v."""
    T, H, d = q.shape
    Hkv = k.shape[1]
    group = H // Hkv
    out = torch.zeros_like(q)
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= (pos[:, None] - pos[None, :]) < window
    for h in range(H):
        kvh = h // group
        s = (q[:, h, :] @ k[:, kvh, :].T) * scale               # [T, T]
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kvh, :]
    return out


def swiglu_mlp(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """crates/metal/examples/qwen2_f16.rs:923-931; crates/kernels/src/cu/ops.cu:111-133:
    h = g / (1 + exp(-g)) * u; out = h Wd^T."""
    g = x @ wg.T
    u = x @ wu.T
    h = g / (1.0 + torch.exp(-g)) * u
    return h @ wd.T


def layer_window(cfg: dict, i: int) -> Optional[int]:
    lt = cfg.get("layer_types")
    if lt is not None:
        return cfg.get("sliding_window") if lt[i] == "sliding_attention" else None
    if cfg.get("use_sliding_window", False) and i >= int(cfg.get("max_window_layers", 0) or 0):
        return cfg.get("sliding_window")
    return None


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict, i: int,
                  positions: torch.Tensor) -> torch.Tensor:
    """crates/metal/examples/qwen2_f16.rs:863-935: norm -> qkv (+bias) -> rope -> attend ->
    Wo -> add -> norm -> swiglu -> add."""
    p = f"model.layers.{i}."
    H = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads") or H
    d = cfg.get("head_dim") or cfg["hidden_size"] // H
    eps = cfg.get("rms_norm_eps", 1e-5)
    theta = cfg.get("rope_theta", 10000.0)
    T = x.shape[0]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = h @ w[p + "self_attn.q_proj.weight"].T
    k = h @ w[p + "self_attn.k_proj.weight"].T
    v = h @ w[p + "self_attn.v_proj.weight"].T
    if p + "self_attn.q_proj.bias" in w:
        q = q + w[p + "self_attn.q_proj.bias"]
        k = k + w[p + "self_attn.k_proj.bias"]
        v = v + w[p + "self_attn.v_proj.bias"]
    rd = int(round(d * cfg.get("partial_rotary_factor", 1.0)))
    q = rope_neox(q.view(T, H, d), positions, theta, rd)
    k = rope_neox(k.view(T, Hkv, d), positions, theta, rd)
    a = attention(q, k, v.view(T, Hkv, d), 1.0 / math.sqrt(d), layer_window(cfg, i))
    x = x + a.reshape(T, H * d) @ w[p + "self_attn.o_proj.weight"].T
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"])
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], token_ids: List[int]) -> torch.Tensor:
    """Logits [T, vocab] for one whole sequence (crates/metal/examples/qwen2_f16.rs:819-939:
    embedding row, layers, final norm, head = lm_head or the embedding when tied)."""
    dev = w["model.embed_tokens.weight"].device       # (a test may hold the weights on a GPU to save time)
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=dev)
    x = w["model.embed_tokens.weight"][ids]
    positions = torch.arange(len(token_ids), device=dev)
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, cfg, i, positions)
    x = rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.T


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int,
                    repetition_penalty: float = 1.0, repetition_window: int = 256) -> List[int]:
    """Argmax continuation, recomputing the whole sequence each step; ties -> lowest index
    (crates/model/src/sampling.rs:302-310).  With a repetition penalty, the logit of every distinct
    token among the last ``repetition_window`` generated ones is divided by it when positive and
    multiplied by it otherwise before the argmax (crates/model/src/sampling.rs:249-277; the logits are
    32-bit there, so the penalised values are rounded to 32-bit here too)."""
    seq = list(prompt)
    out = []
    for _ in range(n):
        logits = forward(cfg, w, seq)[-1]
        if repetition_penalty != 1.0 and out:
            logits = logits.to(torch.float32)
            pen = torch.tensor(repetition_penalty, dtype=torch.float32)
            for t in set(out[-repetition_window:]):
                logits[t] = logits[t] / pen if logits[t] > 0 else logits[t] * pen
        nxt = int(torch.argmax(logits))          # torch.argmax returns the first maximum
        out.append(nxt)
        seq.append(nxt)
    return out
