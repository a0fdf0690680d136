"""Choice of attention kernel for a step.

float32 (the true 32-bit path), head sizes the tensor-core kernels have no instance for, and
page sizes that are no multiple of 16 go to the generic kernel (one warp per token and head).
bf16 steps are split in two: the leading run of single-token requests goes to the split-context
decode kernel, everything after it (prompt portions, and single tokens that follow one) to the
tiled prefill kernel.  The scheduler puts decodes first, as the reference's does
(crates/server/src/scheduler.rs:1037-1041), so that split is the common case.
"""
from __future__ import annotations

from ctypes import byref as _byref, c_float, c_int, c_longlong
from typing import Optional, Sequence, Tuple

import torch

from . import _check, _i32, _ptr, _stream, attention_generic, lib

PREFILL_ROWS = 64          # query rows per CTA of the prefill kernel
MAX_SPLITS = 256           # the merge kernel keeps one weight per split in shared memory


def mma_supported(head_dim: int, page_size: int) -> bool:
    return bool(lib().infero_attn_mma_supported(c_int(head_dim), c_int(page_size)))


def plan_decode(n_tok: int, n_kv: int, group: int, max_visible: int, sm_count: int = 0) -> Tuple[int, int]:
    """(keys per split, number of splits) so that the splits cover ``max_visible`` keys and the
    grid has about two blocks per multiprocessor.  The plan is stated once, in native code
    (``infero_attn_plan_decode``), which the native launcher of a block calls too; ``sm_count`` 0
    means the current device's."""
    chunk, splits = c_int(0), c_int(0)
    lib().infero_attn_plan_decode(c_int(n_tok), c_int(n_kv), c_int(group), c_int(max_visible), c_int(sm_count),
                                  _byref(chunk), _byref(splits))
    return chunk.value, splits.value


_COUNTERS = {}
N_COUNTERS = 1 << 16


def _arrival_counters(device) -> torch.Tensor:
    """Zeroed ints the decode kernel counts finished splits in (every launch leaves them zero)."""
    key = str(device)
    if key not in _COUNTERS:
        _COUNTERS[key] = torch.zeros(N_COUNTERS, dtype=torch.int32, device=device)
    return _COUNTERS[key]


def decode(q, out, k_cache, v_cache, table, tok_entry, positions, tok_first: int, n_tok: int, n_heads: int,
           n_kv: int, head_dim: int, page_size: int, window: Optional[int], scale: float, chunk: int,
           n_splits: int) -> None:
    need = int(lib_scratch(n_tok, n_heads, head_dim, n_splits))
    scratch = torch.empty(need // 4, dtype=torch.float32, device=q.device)
    if lib().infero_attn_decode_tma_supported(c_int(head_dim), c_int(page_size)) and k_cache.is_contiguous() \
            and v_cache.is_contiguous():
        _check(lib().infero_attn_decode_tma(
            _ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
            c_int(k_cache.shape[0]), _ptr(_i32(table, "block_table")), c_int(table.shape[1]),
            _ptr(_i32(tok_entry, "tok_entry")), _ptr(_i32(positions, "positions")), c_int(tok_first), c_int(n_tok),
            c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(page_size), c_int(window or 0), c_float(scale),
            c_int(chunk), c_int(n_splits), _ptr(scratch), _ptr(_arrival_counters(q.device)), c_int(N_COUNTERS),
            _stream()))
        return
    _check(lib().infero_attn_decode(_ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)), _ptr(k_cache),
                                    _ptr(v_cache), _ptr(_i32(table, "block_table")), c_int(table.shape[1]),
                                    _ptr(_i32(tok_entry, "tok_entry")), _ptr(_i32(positions, "positions")),
                                    c_int(tok_first), c_int(n_tok), c_int(n_heads), c_int(n_kv), c_int(head_dim),
                                    c_int(page_size), c_int(window or 0), c_float(scale), c_int(chunk),
                                    c_int(n_splits), _ptr(scratch), _stream()))


def decode_fused(qkv, out, k_cache, v_cache, table, tok_entry, positions, inv_freq, n_heads: int, n_kv: int,
                 head_dim: int, page_size: int, window: Optional[int], scale: float, chunk: int, n_splits: int,
                 write_cache: bool = True, sumsq: Optional[torch.Tensor] = None, sumsq_tiles: int = 0,
                 inv_d: float = 0.0, eps: float = 0.0) -> None:
    """Rotary positions, cache append and decode attention of single tokens in one launch, from the
    q/k/v product as partial sums (``kernels.Partials`` [T, (H + 2 Hkv) * D], bias not yet added)."""
    n_tok = out.shape[0]
    need = int(lib_scratch(n_tok, n_heads, head_dim, n_splits))
    scratch = torch.empty(need // 4, dtype=torch.float32, device=out.device)
    bias = qkv.bias
    _check(lib().infero_attn_decode_tma_fused(
        _ptr(qkv.data), c_int(qkv.splits), c_longlong(qkv.split_stride), _ptr(bias),
        c_int((1 if bias.dtype == torch.bfloat16 else 0) if bias is not None else 0), _ptr(inv_freq),
        c_int(2 * inv_freq.numel()), c_int(1 if write_cache else 0), _ptr(out), c_int(out.stride(0)), _ptr(k_cache),
        _ptr(v_cache), c_int(k_cache.shape[0]), _ptr(_i32(table, "block_table")), c_int(table.shape[1]),
        _ptr(_i32(tok_entry, "tok_entry")), _ptr(_i32(positions, "positions")), c_int(0), c_int(n_tok), c_int(n_heads),
        c_int(n_kv), c_int(head_dim), c_int(page_size), c_int(window or 0), c_float(scale), c_int(chunk),
        c_int(n_splits), _ptr(scratch), _ptr(_arrival_counters(out.device)), c_int(N_COUNTERS), _ptr(sumsq),
        c_int(sumsq_tiles), c_float(inv_d), c_float(eps), _stream()))


def lib_scratch(n_tok, n_heads, head_dim, n_splits) -> int:
    f = lib().infero_attn_decode_scratch
    f.restype = c_longlong
    return f(c_int(n_tok), c_int(n_heads), c_int(head_dim), c_int(n_splits))


def prefill(q, out, k_cache, v_cache, table, entry_q_start, entry_q_len, entry_pos0, n_entries: int,
            first_entry: int, n_tiles: int, n_heads: int, n_kv: int, head_dim: int, page_size: int,
            window: Optional[int], scale: float) -> None:
    _check(lib().infero_attn_prefill(_ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)), _ptr(k_cache),
                                     _ptr(v_cache), _ptr(_i32(table, "block_table")), c_int(table.shape[1]),
                                     _ptr(_i32(entry_q_start, "entry_q_start")), _ptr(_i32(entry_q_len, "entry_q_len")),
                                     _ptr(_i32(entry_pos0, "entry_pos0")), c_int(n_entries), c_int(first_entry),
                                     c_int(n_tiles), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(page_size),
                                     c_int(window or 0), c_float(scale), _stream()))


def prefill_tc_supported(q, out, head_dim: int, page_size: int) -> bool:
    return bool(lib().infero_attn_prefill_tc_supported(c_int(head_dim), c_int(page_size), c_int(q.stride(0)),
                                                       c_int(out.stride(0)))) \
        and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0


def prefill_tc(q, out, k_cache, v_cache, table, entry_q_start, entry_q_len, entry_pos0, n_entries: int,
               first_entry: int, n_tiles: int, n_heads: int, n_kv: int, head_dim: int, page_size: int,
               window: Optional[int], scale: float) -> None:
    """The tcgen05 kernel: 128 query rows per block (n_tiles counts blocks of 128)."""
    _check(lib().infero_attn_prefill_tc(
        _ptr(q), c_int(q.stride(0)), c_int(q.shape[0]), _ptr(out), c_int(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(k_cache.shape[0]), _ptr(_i32(table, "block_table")), c_int(table.shape[1]),
        _ptr(_i32(entry_q_start, "entry_q_start")), _ptr(_i32(entry_q_len, "entry_q_len")),
        _ptr(_i32(entry_pos0, "entry_pos0")), c_int(n_entries), c_int(first_entry), c_int(n_tiles), c_int(n_heads),
        c_int(n_kv), c_int(head_dim), c_int(page_size), c_int(window or 0), c_float(scale), _stream()))


def shape_of_batch(q_lens: Sequence[int], pos0: Sequence[int]):
    """What the choice of kernels needs to know of a batch, the same for every layer of a step:
    (single-token requests in front, most keys any of them sees, blocks of 128 query rows of the
    others, blocks of the mma.sync kernel's height)."""
    E = len(q_lens)
    n_dec = 0
    while n_dec < E and q_lens[n_dec] == 1:
        n_dec += 1
    vis = max((int(pos0[i]) + 1 for i in range(n_dec)), default=0)
    tiles_128 = sum(-(-int(n) // 128) for n in q_lens[n_dec:])
    tiles_mma = sum(-(-int(n) // PREFILL_ROWS) for n in q_lens[n_dec:])
    return n_dec, vis, tiles_128, tiles_mma


def attention_any(q, out, k_cache, v_cache, table, tok_entry, positions, n_heads: int, n_kv: int, head_dim: int,
                  page_size: int, window: Optional[int], scale: float, q_lens: Sequence[int], pos0: Sequence[int],
                  entry_q_start=None, entry_q_len=None, entry_pos0=None, kv_bound: Optional[int] = None,
                  batch_shape=None) -> None:
    """q: [T, >= H*D] view with rotated queries in front (row stride free); out [T, H*D].
    ``q_lens`` / ``pos0`` are the host copies of each request's new-token count and cached
    length; the device copies are made here when the caller has none.  ``kv_bound``: plan the
    decode splits for this many visible keys instead of what the batch holds now (a captured
    step is replayed while its requests grow)."""
    if q.dtype != torch.bfloat16 or not mma_supported(head_dim, page_size):
        attention_generic(q, out, k_cache, v_cache, table, tok_entry, positions, n_heads, n_kv, head_dim,
                          page_size, window, scale)
        return
    E = len(q_lens)
    if batch_shape is None:
        batch_shape = shape_of_batch(q_lens, pos0)
    n_dec, vis_now, tiles_128, tiles_mma = batch_shape
    if n_dec:
        vis = vis_now if kv_bound is None else int(kv_bound)
        if window:
            vis = min(vis, window + 15)
        chunk, splits = plan_decode(n_dec, n_kv, n_heads // n_kv, vis)
        decode(q, out, k_cache, v_cache, table, tok_entry, positions, 0, n_dec, n_heads, n_kv, head_dim,
               page_size, window, scale, chunk, splits)
    if n_dec < E:
        if entry_q_len is None:
            dev = q.device
            starts = [0]
            for n in q_lens[:-1]:
                starts.append(starts[-1] + int(n))
            entry_q_start = torch.tensor(starts, dtype=torch.int32, device=dev)
            entry_q_len = torch.tensor([int(n) for n in q_lens], dtype=torch.int32, device=dev)
            entry_pos0 = torch.tensor([int(p) for p in pos0], dtype=torch.int32, device=dev)
        if prefill_tc_supported(q, out, head_dim, page_size) and k_cache.is_contiguous() and v_cache.is_contiguous():
            n_tiles = tiles_128
            prefill_tc(q, out, k_cache, v_cache, table, entry_q_start, entry_q_len, entry_pos0, E, n_dec, n_tiles,
                       n_heads, n_kv, head_dim, page_size, window, scale)
            return
        n_tiles = tiles_mma
        prefill(q, out, k_cache, v_cache, table, entry_q_start, entry_q_len, entry_pos0, E, n_dec, n_tiles,
                n_heads, n_kv, head_dim, page_size, window, scale)


def paged_attention(ctx, qkv, out, kv, table, n_heads, n_kv, head_dim, window, scale) -> None:
    """qkv: [T, (H + 2 Hkv) D] with rotated queries in front; out [T, H*D]."""
    attention_any(qkv, out, kv.k, kv.v, table, ctx.tok_entry, ctx.positions, n_heads, n_kv, head_dim,
                  kv.page_size, window, scale, ctx.h_q_len, ctx.h_pos0, ctx.entry_q_start, ctx.entry_q_len,
                  ctx.entry_pos0, kv_bound=getattr(ctx, "kv_bound", None), batch_shape=_batch_shape(ctx))


def _batch_shape(ctx):
    memo = getattr(ctx, "_attn_batch_shape", None)
    if memo is None:
        memo = shape_of_batch(ctx.h_q_len, ctx.h_pos0)
        try:
            ctx._attn_batch_shape = memo
        except AttributeError:          # a context that takes no new attributes
            pass
    return memo
