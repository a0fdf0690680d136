"""Python face of the CUDA library: thin wrappers that check tensors and call the exported
C launchers on the current torch stream.

There is no CPU path and no library model code behind these names: if the shared library
cannot be built or loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_float, c_void_p, c_char_p, POINTER
from typing import Optional

import torch

from .build import ensure_built, BuildError

F32, BF16 = 0, 1
_LIB = None


class KernelError(RuntimeError):
    pass


def lib():
    """The loaded shared library (built on first use)."""
    global _LIB
    if _LIB is None:
        path = ensure_built()
        try:
            L = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from None
        L.infero_last_error.restype = c_char_p
        L.infero_abi_version.restype = c_int
        _LIB = L
    return _LIB


def launch_count() -> int:
    """Kernels launched through this library so far (a launch recorded into a CUDA graph
    counts once, when it is captured)."""
    f = lib().infero_launch_count
    f.restype = ctypes.c_longlong
    return int(f())


def loaded_library_path() -> Optional[str]:
    return None if _LIB is None else _LIB._name


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported tensor dtype {t.dtype} (float32 or bfloat16 only)")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("tensor is not on a CUDA device; this engine has no CPU path")
    return c_void_p(t.data_ptr())


_SCOPED_STREAM: Optional[c_void_p] = None


def _stream() -> c_void_p:
    """The stream kernels are launched on: torch's current stream, looked up once per
    ``stream_scope`` (a look-up costs about as much as a launch) or at every call outside one."""
    if _SCOPED_STREAM is not None:
        return _SCOPED_STREAM
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Inside, every kernel of this module goes to the stream that was current on entry (enter it
    inside ``torch.cuda.graph`` / ``torch.cuda.stream``, not around them)."""

    def __enter__(self):
        global _SCOPED_STREAM
        self._prev = _SCOPED_STREAM
        _SCOPED_STREAM = c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _SCOPED_STREAM
        _SCOPED_STREAM = self._prev
        return False


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(lib().infero_last_error().decode("utf-8", "replace"))


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return t


# ---- embedding, norms, elementwise ---------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out_x: torch.Tensor, scale: float = 1.0,
                 device_tokens: Optional[torch.Tensor] = None) -> None:
    """out_x[t,:] = table[ids[t],:] * scale, out_x float32 [T, d].  An id -(s + 1) is replaced
    by device_tokens[s] (the token a sampler left on the device) when that array is given."""
    T, d = out_x.shape
    assert out_x.dtype == torch.float32 and out_x.is_contiguous() and table.is_contiguous()
    assert table.shape[1] == d and ids.numel() == T
    _check(lib().infero_embed_gather(_ptr(table), c_int(_dt(table)), _ptr(_i32(ids, "ids")),
                                     _ptr(None if device_tokens is None else _i32(device_tokens, "device_tokens")),
                                     _ptr(out_x), c_int(T), c_int(d), c_int(table.shape[0]), c_float(scale), _stream()))


class Partials:
    """A matrix product left as 32-bit partial sums: the value is sum_s data[s] (+ bias), s in
    ascending order.  The few-token tensor-core kernel writes these; the kernel that consumes
    the product (norm, activation, rotary + cache append) adds them up in its own pass."""

    def __init__(self, data: torch.Tensor, bias: Optional[torch.Tensor] = None):
        assert data.dim() == 3 and data.dtype == torch.float32 and data.is_contiguous()
        self.data = data
        self.bias = bias

    @property
    def shape(self):
        return self.data.shape[1:]

    @property
    def splits(self) -> int:
        return self.data.shape[0]

    @property
    def split_stride(self) -> int:
        return self.data.shape[1] * self.data.shape[2]

    def materialize(self, dtype: torch.dtype) -> torch.Tensor:
        """The value as one tensor (for parts that have no fused kernel of their own)."""
        from .tc_gemm import reduce_partials
        out = torch.empty(tuple(self.shape), dtype=dtype, device=self.data.device)
        reduce_partials(self.data, self.bias, out)
        return out


def add_rmsnorm(x: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """x += delta (if given; 32-bit), out = rmsnorm(x) * weight.  ``delta`` is a tensor or
    ``Partials``.  With ``rows`` only those rows are normalised (out has len(rows) rows) and x
    is left as it is."""
    if hasattr(delta, "as_partials"):          # left by the native block launcher in its scratch arena
        delta = delta.as_partials()
    d = x.shape[1]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    assert weight.numel() == d and out.shape[1] == d
    n = out.shape[0]
    if rows is None:
        assert n == x.shape[0]
    else:
        assert rows.numel() == n
    splits, stride, dbias, data = 1, 0, None, delta
    if isinstance(delta, Partials):
        data, splits, stride, dbias = delta.data, delta.splits, delta.split_stride, delta.bias
        assert tuple(delta.shape) == tuple(x.shape)
    elif delta is not None:
        assert delta.shape == x.shape and delta.is_contiguous()
    _check(lib().infero_add_rmsnorm(_ptr(x), _ptr(data), c_int(_dt(data) if data is not None else F32),
                                    c_int(splits), ctypes.c_longlong(stride), _ptr(dbias),
                                    c_int(_dt(dbias) if dbias is not None else F32),
                                    _ptr(weight), c_int(_dt(weight)), c_float(eps), _ptr(out), c_int(_dt(out)),
                                    _ptr(None if rows is None else _i32(rows, "rows")), c_int(n), c_int(d),
                                    _stream()))


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    assert x.dtype == torch.float32 and x.shape == delta.shape and x.is_contiguous() and delta.is_contiguous()
    _check(lib().infero_residual_add(_ptr(x), _ptr(delta), c_int(_dt(delta)), c_int(x.shape[0]),
                                     c_int(x.shape[1]), _stream()))


def swiglu(gate_up, out: torch.Tensor) -> None:
    """out[t, j] = silu(g[t, 2j]) * g[t, 2j + 1] for g = gate_up (a tensor of out's type, or
    ``Partials`` with a bf16 out): gate and up alternate along a row."""
    T, ff = out.shape
    assert out.is_contiguous()
    if isinstance(gate_up, Partials):
        assert tuple(gate_up.shape) == (T, 2 * ff) and gate_up.bias is None and out.dtype == torch.bfloat16
        _check(lib().infero_swiglu(_ptr(gate_up.data), c_int(gate_up.splits), ctypes.c_longlong(gate_up.split_stride),
                                   _ptr(out), c_int(F32), c_int(1), c_int(T), c_int(ff), _stream()))
        return
    assert gate_up.shape == (T, 2 * ff) and gate_up.dtype == out.dtype and gate_up.is_contiguous()
    _check(lib().infero_swiglu(_ptr(gate_up), c_int(1), ctypes.c_longlong(0), _ptr(out), c_int(_dt(out)), c_int(0),
                               c_int(T), c_int(ff), _stream()))


# ---- matrix products ------------------------------------------------------------------------
def gemm_tiled(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias); 32-bit accumulation in ascending k."""
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and w.is_contiguous()
    assert a.stride(1) == 1 and out.stride(1) == 1
    _check(lib().infero_gemm_tiled(_ptr(a), c_int(_dt(a)), _ptr(w), c_int(_dt(w)), _ptr(bias),
                                   c_int(_dt(bias) if bias is not None else F32), _ptr(out), c_int(_dt(out)),
                                   c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), c_int(out.stride(0)),
                                   _stream()))


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """bf16 x bf16 for 1..4 rows of a."""
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous()
    assert w.shape[1] == K and out.shape == (M, N) and a.stride(1) == 1 and out.stride(1) == 1
    _check(lib().infero_gemm_skinny(_ptr(a), _ptr(w), _ptr(bias), c_int(_dt(bias) if bias is not None else F32),
                                    _ptr(out), c_int(_dt(out)), c_int(M), c_int(N), c_int(K),
                                    c_int(a.stride(0)), c_int(out.stride(0)), _stream()))


# ---- position encoding + cache append, attention --------------------------------------------
def rope_cache(qkv: torch.Tensor, positions: torch.Tensor, tok_entry: torch.Tensor, block_table: torch.Tensor,
               inv_freq: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int, n_kv: int,
               head_dim: int, page_size: int, write_cache: bool = True) -> None:
    """Rotate q (in place) and k, append k and v to their pages.  qkv [T, (H + 2 Hkv) * D];
    caches [pages, Hkv, page_size, D] of qkv's dtype; block_table [entries, max_blocks]."""
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == (n_heads + 2 * n_kv) * head_dim
    assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and block_table.dim() == 2
    assert inv_freq.dtype == torch.float32
    rotary = 2 * inv_freq.numel()
    _check(lib().infero_rope_cache(_ptr(qkv), c_int(_dt(qkv)), c_int(qkv.stride(0)), _ptr(_i32(positions, "positions")),
                                   _ptr(_i32(tok_entry, "tok_entry")), _ptr(_i32(block_table, "block_table")),
                                   c_int(block_table.shape[1]), _ptr(inv_freq), c_int(rotary), _ptr(k_cache),
                                   _ptr(v_cache), c_int(page_size), c_int(T), c_int(n_heads), c_int(n_kv),
                                   c_int(head_dim), c_int(1 if write_cache else 0), _stream()))


def rope_cache_partials(qkv: Partials, q_out: torch.Tensor, positions: torch.Tensor, tok_entry: torch.Tensor,
                        block_table: torch.Tensor, inv_freq: torch.Tensor, k_cache: torch.Tensor,
                        v_cache: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, page_size: int,
                        write_cache: bool = True) -> None:
    """The same from partial sums (+ bias): rotated q goes to q_out [T, H * D], k and v to their pages."""
    T = q_out.shape[0]
    assert tuple(qkv.shape) == (T, (n_heads + 2 * n_kv) * head_dim) and q_out.stride(1) == 1
    assert q_out.shape[1] == n_heads * head_dim and k_cache.dtype == q_out.dtype == v_cache.dtype
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and inv_freq.dtype == torch.float32
    _check(lib().infero_rope_cache_partials(
        _ptr(qkv.data), c_int(qkv.splits), ctypes.c_longlong(qkv.split_stride), _ptr(qkv.bias),
        c_int(_dt(qkv.bias) if qkv.bias is not None else F32), _ptr(q_out), c_int(q_out.stride(0)),
        c_int(_dt(q_out)), _ptr(_i32(positions, "positions")), _ptr(_i32(tok_entry, "tok_entry")),
        _ptr(_i32(block_table, "block_table")), c_int(block_table.shape[1]), _ptr(inv_freq),
        c_int(2 * inv_freq.numel()), _ptr(k_cache), _ptr(v_cache), c_int(page_size), c_int(T), c_int(n_heads),
        c_int(n_kv), c_int(head_dim), c_int(1 if write_cache else 0), _stream()))


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_table: torch.Tensor, tok_entry: torch.Tensor, positions: torch.Tensor,
                      n_heads: int, n_kv: int, head_dim: int, page_size: int, window: Optional[int],
                      scale: float) -> None:
    """q: [T, >= H*D] view (row stride free), out [T, H*D]."""
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_cache.dtype
    _check(lib().infero_attention_generic(_ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)),
                                          _ptr(k_cache), _ptr(v_cache), c_int(_dt(q)),
                                          _ptr(_i32(block_table, "block_table")), c_int(block_table.shape[1]),
                                          _ptr(_i32(tok_entry, "tok_entry")), _ptr(_i32(positions, "positions")),
                                          c_int(T), c_int(n_heads), c_int(n_kv), c_int(head_dim),
                                          c_int(page_size), c_int(window or 0), c_float(scale), _stream()))


# ---- sampling --------------------------------------------------------------------------------
def apply_penalty(logits: torch.Tensor, pen_tokens: torch.Tensor, pen_counts: torch.Tensor,
                  penalty: torch.Tensor) -> None:
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and penalty.dtype == torch.float32
    assert pen_tokens.shape == pen_counts.shape and pen_tokens.shape[0] == R
    _check(lib().infero_apply_penalty(_ptr(logits), c_int(R), c_int(V), _ptr(_i32(pen_tokens, "pen_tokens")),
                                      _ptr(_i32(pen_counts, "pen_counts")), c_int(pen_tokens.shape[1]),
                                      _ptr(penalty), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and out.numel() >= R
    f = lib().infero_argmax_scratch
    f.restype = ctypes.c_longlong
    scratch = torch.empty(int(f(c_int(R), c_int(V))) // 4, dtype=torch.float32, device=logits.device)
    _check(lib().infero_argmax(_ptr(logits), c_int(R), c_int(V), _ptr(_i32(out, "out")), _ptr(scratch), _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           draw: torch.Tensor, out: torch.Tensor) -> None:
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and draw.dtype == torch.float64
    L = lib()
    L.infero_sample_scratch.restype = ctypes.c_longlong
    need = int(L.infero_sample_scratch(c_int(R), c_int(V)))
    scratch = torch.empty(need // 8, dtype=torch.int64, device=logits.device) if need else None
    _check(L.infero_sample(_ptr(logits), c_int(R), c_int(V), _ptr(temperature), _ptr(_i32(top_k, "top_k")),
                           _ptr(top_p), _ptr(draw), _ptr(_i32(out, "out")), _ptr(scratch), ctypes.c_longlong(need),
                           _stream()))


def keep_tokens(greedy: torch.Tensor, sampled: Optional[torch.Tensor], rows_info: torch.Tensor,
                final_tok: torch.Tensor, device_tokens: torch.Tensor, ring: Optional[torch.Tensor] = None,
                ring_len: Optional[torch.Tensor] = None, with_fault: bool = False) -> None:
    """final_tok[r] = sampled[r] if rows_info[R + r] else greedy[r]; device_tokens[rows_info[r]] = final_tok[r];
    with ``ring`` [slots, width] / ``ring_len`` [slots] the pick is appended to its request's history.
    ``with_fault``: final_tok has one more element, which receives the device's fault flag (the one the
    kernels with bounded waits raise), so the host reads it with the picks."""
    R = final_tok.numel() - (1 if with_fault else 0)
    assert rows_info.numel() == 2 * R and (ring is None) == (ring_len is None)
    _check(lib().infero_keep_tokens(_ptr(_i32(greedy, "greedy")), _ptr(None if sampled is None else _i32(sampled, "sampled")),
                                    _ptr(_i32(rows_info, "rows_info")), _ptr(_i32(final_tok, "final_tok")),
                                    _ptr(_i32(device_tokens, "device_tokens")), c_int(R),
                                    _ptr(None if ring is None else _i32(ring, "ring")),
                                    _ptr(None if ring_len is None else _i32(ring_len, "ring_len")),
                                    c_int(ring.shape[1] if ring is not None else 0), c_int(1 if with_fault else 0),
                                    _stream()))


def apply_penalty_ring(logits: torch.Tensor, rows_info: torch.Tensor, penalty: torch.Tensor, window: torch.Tensor,
                       ring: torch.Tensor, ring_len: torch.Tensor) -> None:
    """The repetition penalty from the histories kept on the device (``keep_tokens`` appends to them):
    row r looks at the last ``window[r]`` tokens of request slot ``rows_info[r]``."""
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and penalty.dtype == torch.float32
    assert rows_info.numel() == 2 * R and ring.dim() == 2 and ring.is_contiguous()
    _check(lib().infero_apply_penalty_ring(_ptr(logits), c_int(R), c_int(V), _ptr(_i32(rows_info, "rows_info")),
                                           _ptr(penalty), _ptr(_i32(window, "window")), _ptr(_i32(ring, "ring")),
                                           _ptr(_i32(ring_len, "ring_len")), c_int(ring.shape[1]), _stream()))


def sample_max_k() -> int:
    return int(lib().infero_sample_max_k())
