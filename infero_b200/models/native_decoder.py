"""The whole model launched by native code in one call per step.

When every execution of a model's schedule is a built-in block that goes the native way
(``parts/native_block.py``), its final norm is the package's RMSNorm and its output product runs on the
tensor-core kernel, ``DecoderModel.forward`` hands the step to ``infero_decoder_forward``
(``csrc/host_block.cpp``): embedding, the blocks, the final norm on the wanted rows and the output product,
launch for launch what the Python loop does (the same native functions with the same arguments, so the
logits are the same bit for bit).  The host's share of a step that is not replayed from a CUDA graph drops
from a Python call per layer to one call; ``INFERO_NATIVE_STEP=0`` keeps the loop.

The reference runs its whole pass natively (crates/model/src/lib.rs:3423-4243).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .. import kernels as K
from ..kernels import tc_gemm
from ..parts import native_block as NB

ENABLED = os.environ.get("INFERO_NATIVE_STEP", "1") != "0"
CALLS = [0]                 # steps run this way so far (tests look at it)


def set_enabled(on: bool) -> None:
    global ENABLED
    ENABLED = bool(on)


class _Decoder(ctypes.Structure):
    _fields_ = [("n_entries", c_int), ("blocks", c_void_p), ("entry_group", c_void_p), ("embed", c_void_p),
                ("embed_dtype", c_int), ("vocab", c_int), ("hidden", c_int), ("embed_scale", c_float),
                ("final_norm_w", c_void_p), ("final_norm_dtype", c_int), ("final_eps", c_float),
                ("head_w", c_void_p), ("head_bias", c_void_p), ("head_bias_dtype", c_int)]


class NativeDecoder:
    """Built once per ``DecoderModel``; ``run`` is its ``forward`` (or says that this step cannot go this way)."""

    def __init__(self, model):
        self.model = model
        self._per_pool = {}          # id(cache storage) -> (storage, _Decoder, what it points to)
        self.ok = self._qualifies()

    def _qualifies(self) -> bool:
        from ..parts.block import PreNormBlock
        from ..parts.norm import RmsNorm
        m = self.model
        if m.spec.logit_scale != 1.0 or type(m.final_norm) is not RmsNorm:
            return False
        if not all(type(b) is PreNormBlock for b in m.blocks):
            return False
        head = m.head
        return head.weight.dtype == torch.bfloat16 and head.weight.is_cuda and m.embed.is_cuda

    def _descriptor(self, ctx):
        """The model as native code takes it, for the cache pool of this step's runner."""
        storage = ctx._runner.storage
        hit = self._per_pool.get(id(storage))
        if hit is not None and hit[0] is storage:
            return hit[1]
        m, s = self.model, self.model.spec
        descs, groups = [], []
        for entry in s.schedule:
            nb = m.blocks[entry.block]._native_for(ctx)
            d = nb._desc(ctx, entry) if nb is not None else None
            if d is None:
                self._per_pool[id(storage)] = (storage, None, None)
                return None
            descs.append(d)
            groups.append(int(ctx.kv_cache(entry.cache).group))
        blocks = (NB._Block * len(descs))(*descs)
        entry_group = (c_int * len(groups))(*groups)
        ptr = lambda t: t.data_ptr() if t is not None else None     # noqa: E731
        head = m.head
        dec = _Decoder(len(descs), ctypes.cast(blocks, c_void_p), ctypes.cast(entry_group, c_void_p), ptr(m.embed),
                       NB._dt(m.embed), int(s.vocab_size), int(s.hidden), float(s.embed_scale), ptr(m.final_norm.weight),
                       NB._dt(m.final_norm.weight), float(m.final_norm.spec.eps), ptr(head.weight), ptr(head.bias),
                       NB._dt(head.bias))
        self._per_pool[id(storage)] = (storage, dec, (blocks, entry_group, descs))
        return dec

    def run(self, ctx, token_ids: torch.Tensor, logit_rows: Optional[torch.Tensor]):
        """Logits [rows, vocab] (None when no row is wanted), or NotImplemented when this step has to take
        the Python loop after all."""
        if not (ENABLED and NB.ENABLED and self.ok) or getattr(ctx, "act_dtype", None) != torch.bfloat16:
            return NotImplemented
        if getattr(ctx, "_runner", None) is None or getattr(ctx, "h_q_len", None) is None:
            return NotImplemented
        dec = self._descriptor(ctx)
        if dec is None:
            return NotImplemented
        m, s = self.model, self.model.spec
        T = token_ids.numel()
        R = 0 if logit_rows is None else logit_rows.numel()
        dev = token_ids.device
        x = torch.empty((T, s.hidden), dtype=torch.float32, device=dev)
        h_rows = torch.empty((max(R, 1), s.hidden), dtype=torch.bfloat16, device=dev)
        logits = torch.empty((R, s.vocab_size), dtype=torch.float32, device=dev) if R else None
        if R and not tc_gemm.supported(h_rows[:R], m.head.weight, logits):
            return NotImplemented
        descs = self._per_pool[id(ctx._runner.storage)][2][2]
        for d in descs:                                  # the scratch arena grows to what the largest block needs
            if ctx._runner.native_arena(d) is None:
                return NotImplemented
        step = ctx.native_step(x, descs[0])
        if step is None:
            return NotImplemented
        ws_bytes = tc_gemm.plan(R, s.vocab_size, s.hidden, dev)[2] if 0 < R <= 256 else 0
        ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device=dev) if ws_bytes else None
        n_groups = len(ctx._tables)
        tables = (c_void_p * n_groups)(*[ctx.block_table(g).data_ptr() for g in range(n_groups)])
        device_tokens = getattr(ctx, "device_tokens", None)
        K._check(NB._lib().infero_decoder_forward(
            ctypes.byref(dec), ctypes.byref(step), K._ptr(K._i32(token_ids, "token_ids")),
            K._ptr(None if device_tokens is None else K._i32(device_tokens, "device_tokens")), tables,
            c_int(ctx.block_table(0).shape[1]), K._ptr(None if not R else K._i32(logit_rows, "rows")), c_int(R),
            K._ptr(h_rows), K._ptr(logits), K._ptr(ws), c_longlong(ws_bytes)))
        NB.CALLS[0] += dec.n_entries
        CALLS[0] += 1
        ctx._native_keep_step = (x, h_rows, ws)          # alive until the step's kernels have run
        return logits
