"""The built-in block launched by native code in one call per layer.

``PreNormBlock`` made of exactly the package's own parts (RMSNorm, grouped-query attention with
NeoX rotary positions or none, SwiGLU) in a bf16 step can hand its whole layer to
``infero_block_forward`` (``csrc/host_block.cpp``).  In steps with a prompt portion that call launches
the same kernels with the same arguments in the same order as the parts launch one by one, so the
results are the same bit for bit; what changes is the host's time per layer (one call instead of a
dozen wrappers), which is what bounds steps that are not replayed from a CUDA graph.  In steps of
single tokens the native layer is made of fewer launches than the parts' (decode attention finishes
the q/k/v product itself; the norms are folded into the products around them, see ``set_fusion``).
Any other block, dtype or part keeps to the parts' own ``forward``.  ``INFERO_NATIVE_BLOCK=0`` turns
it off.

The reference runs its layer loop natively throughout (crates/model/src/lib.rs:3423-4243).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .. import kernels as K

ENABLED = os.environ.get("INFERO_NATIVE_BLOCK", "1") != "0"
CALLS = [0]                 # layers run natively so far (tests look at it)


def set_enabled(on: bool) -> None:
    """Switch for blocks built from now on and for those that exist (checked at every layer)."""
    global ENABLED
    ENABLED = bool(on)


def set_fusion(decode: bool = True, norms: bool = True) -> None:
    """Steps of single tokens: ``decode``: attention finishes the q/k/v product itself (bias, rotary
    positions, cache append; bit for bit what the separate kernels give); ``norms``: the residual-add-and-
    norm kernels are folded into the products around them (same arithmetic up to where bf16 rounding
    falls).  Both on unless INFERO_FUSED_DECODE=0 / INFERO_FUSED_NORM=0."""
    _lib().infero_block_set_fusion(c_int(1 if decode else 0), c_int(1 if norms else 0))


F32, BF16 = K.F32, K.BF16
PRENORMED = 2               # a pending output that is no longer pending: see InferoDelta in csrc/host_block.cpp


class _Block(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("hidden", "n_heads", "n_kv", "head_dim", "intermediate", "rotary_dim", "window",
                                     "write_cache")] + \
               [(n, c_float) for n in ("eps_mixer", "eps_ffn", "scale")] + \
               [(n, c_int) for n in ("norm_dtype", "qkv_bias_dtype", "o_bias_dtype")] + \
               [(n, c_void_p) for n in ("w_norm_mixer", "w_norm_ffn", "w_qkv", "b_qkv", "w_o", "b_o", "w_gate_up",
                                        "w_down", "inv_freq", "k_cache", "v_cache")] + \
               [(n, c_int) for n in ("num_pages", "page_size")]


class _Step(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("n_tokens", "n_entries", "n_decode", "decode_visible", "prefill_tiles",
                                     "sm_count")] + \
               [(n, c_void_p) for n in ("positions", "tok_entry", "entry_q_start", "entry_q_len", "entry_pos0", "x",
                                        "arena")] + \
               [("arena_bytes", c_longlong), ("counters", c_void_p), ("n_counters", c_int), ("stream", c_void_p)]


class _Delta(ctypes.Structure):
    _fields_ = [("data", c_void_p), ("dtype", c_int), ("splits", c_int), ("split_stride", c_longlong),
                ("bias", c_void_p), ("bias_dtype", c_int), ("sumsq", c_void_p), ("sumsq_tiles", c_int)]


def _lib():
    L = K.lib()
    if not getattr(L, "_block_api_ready", False):
        L.infero_block_arena_bytes.restype = c_longlong
        L._block_api_ready = True
    return L


def _dt(t: Optional[torch.Tensor]) -> int:
    return F32 if t is None or t.dtype == torch.float32 else BF16


class NativeDelta:
    """A layer's pending output where native code left it (in the step's scratch arena).  The next
    native layer takes the descriptor as it is; a Python consumer asks for ``as_partials()``."""

    def __init__(self, desc: _Delta, arena: torch.Tensor, rows: int, cols: int, bias: Optional[torch.Tensor]):
        self.desc, self.arena, self.rows, self.cols, self.bias_tensor = desc, arena, rows, cols, bias

    def as_partials(self):
        if self.desc.dtype == PRENORMED:
            return None                        # x holds the sum already: nothing is pending for a Python consumer
        off = int(self.desc.data) - self.arena.data_ptr()
        if self.desc.dtype == F32:
            n = self.desc.splits * self.rows * self.cols
            data = self.arena[off:off + 4 * n].view(torch.float32).view(self.desc.splits, self.rows, self.cols)
            return K.Partials(data, self.bias_tensor)
        return self.arena[off:off + 2 * self.rows * self.cols].view(torch.bfloat16).view(self.rows, self.cols)


def _delta_desc(delta, keep: list) -> _Delta:
    """The descriptor of whatever the layer before left pending."""
    if delta is None:
        return _Delta(None, F32, 1, 0, None, F32, None, 0)
    if isinstance(delta, NativeDelta):
        return delta.desc
    if isinstance(delta, K.Partials):
        keep.append(delta)
        b = delta.bias
        return _Delta(delta.data.data_ptr(), F32, delta.splits, delta.split_stride, b.data_ptr() if b is not None else None,
                      _dt(b), None, 0)
    if not delta.is_contiguous():
        delta = delta.contiguous()
    keep.append(delta)
    return _Delta(delta.data_ptr(), _dt(delta), 1, 0, None, F32, None, 0)


class NativeBlock:
    """Built once per ``PreNormBlock`` that qualifies; ``run`` is its ``forward``."""

    def __init__(self, block):
        self.block = block
        self._descs = {}                   # (cache slot, write_cache) -> (_Block, the pool it points into, inv_freq)
        self.ok = self._parts_qualify()

    # ---- which blocks -----------------------------------------------------------------------
    def _parts_qualify(self) -> bool:
        from .attention import GqaAttention
        from .mlp import SwiGluMlp
        from .norm import RmsNorm
        from .rope import RopeNeox
        b = self.block
        if type(b.mixer) is not GqaAttention or type(b.ffn) is not SwiGluMlp:
            return False
        if type(b.mixer_norm) is not RmsNorm or type(b.ffn_norm) is not RmsNorm:
            return False
        if b.mixer.rope is not None and type(b.mixer.rope) is not RopeNeox:
            return False
        return True

    def _weights_qualify(self) -> bool:
        b = self.block
        mats = (b.mixer.qkv, b.mixer.out, b.ffn.gate_up, b.ffn.down)
        if any(m is None or m.weight.dtype != torch.bfloat16 or not m.weight.is_cuda for m in mats):
            return False
        if b.ffn.gate_up.bias is not None or b.ffn.down.bias is not None:
            return False
        w1, w2 = b.mixer_norm.weight, b.ffn_norm.weight
        return w1 is not None and w2 is not None and w1.dtype == w2.dtype and w1.dtype in (torch.float32, torch.bfloat16)

    def wants(self, ctx) -> bool:
        """Does this step go the native way?  (A bf16 step of a runner, on bf16 weights.)"""
        if not ENABLED or not self.ok or getattr(ctx, "act_dtype", None) != torch.bfloat16 or getattr(ctx, "_runner", None) is None:
            return False
        if not hasattr(self, "_weights_ok"):
            self._weights_ok = self._weights_qualify()
        return self._weights_ok

    # ---- descriptors -------------------------------------------------------------------------
    def _desc(self, ctx, slot):
        key = (slot.cache, bool(slot.write_cache))
        kv = ctx.kv_cache(slot.cache)
        hit = self._descs.get(key)
        if hit is not None and hit[1] is kv:       # the same pool as last time (a model may serve several runners)
            return hit[0]
        b, m = self.block, self.block.mixer.spec
        if kv.k.dtype != torch.bfloat16 or not kv.k.is_contiguous() or not kv.v.is_contiguous():
            self._descs[key] = (None, kv, None)
            return None
        rope = self.block.mixer.rope
        inv = rope.inv_freq(kv.k.device) if rope is not None else None
        qkv, out, gu, down = b.mixer.qkv, b.mixer.out, b.ffn.gate_up, b.ffn.down
        ptr = lambda t: t.data_ptr() if t is not None else None     # noqa: E731
        d = _Block(m.hidden, m.num_heads, m.num_kv_heads, m.head_dim, b.ffn.spec.intermediate,
                   2 * inv.numel() if inv is not None else 0, int(m.window or 0), int(bool(slot.write_cache)),
                   float(b.mixer_norm.spec.eps), float(b.ffn_norm.spec.eps), float(m.scale),
                   _dt(b.mixer_norm.weight), _dt(qkv.bias), _dt(out.bias),
                   ptr(b.mixer_norm.weight), ptr(b.ffn_norm.weight), ptr(qkv.weight), ptr(qkv.bias), ptr(out.weight),
                   ptr(out.bias), ptr(gu.weight), ptr(down.weight), ptr(inv), ptr(kv.k), ptr(kv.v),
                   int(kv.k.shape[0]), int(kv.page_size))
        if not _lib().infero_block_supported(ctypes.byref(d)):
            d = None
        self._descs[key] = (d, kv, inv)
        return d

    # ---- the layer -----------------------------------------------------------------------------
    def run(self, ctx, x, delta, slot):
        """None when this execution cannot go the native way after all (the caller then runs the parts)."""
        d = self._desc(ctx, slot)
        if d is None:
            return None
        step = ctx.native_step(x, d)
        if step is None:
            return None
        kv = ctx.kv_cache(slot.cache)
        table = ctx.block_table(kv.group)
        keep = []
        desc = _delta_desc(delta, keep)
        out = _Delta(desc.data, desc.dtype, desc.splits, desc.split_stride, desc.bias, desc.bias_dtype, desc.sumsq,
                     desc.sumsq_tiles)
        parity = ctx.native_parity
        ctx.native_parity ^= 1
        # the block that runs next on the same residual stream, if it is one of these too: native code may
        # then fold that block's first norm into this block's last product
        nxt = None
        upcoming = getattr(ctx, "upcoming", None)
        if upcoming is not None:
            nb = getattr(upcoming[0], "_native_for", lambda c: None)(ctx)
            if nb is not None:
                nxt = nb._desc(ctx, upcoming[1])
        K._check(_lib().infero_block_forward(ctypes.byref(d), ctypes.byref(step), c_void_p(table.data_ptr()),
                                             c_int(table.shape[1]), c_int(parity), ctypes.byref(out),
                                             ctypes.byref(nxt) if nxt is not None else None))
        CALLS[0] += 1
        return NativeDelta(out, ctx.native_arena, x.shape[0], d.hidden, None)
