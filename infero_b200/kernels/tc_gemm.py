"""Tensor-core (tcgen05 / TMEM / TMA) matrix product for bf16 operands.

``gemm`` computes out = a @ w^T (+ bias).  With few rows (<= 256) the weights take the
128-wide side of the MMA and K is cut into splits so that every SM streams weights; the
32-bit partial products go through a workspace and are summed in a fixed order.
``partials`` exposes those partial products to consumers that fold the sum into their own
pass (norm, activation, rotary + cache append).
"""
from __future__ import annotations

from ctypes import byref, c_int, c_longlong
from typing import Optional, Tuple

import torch

from . import F32, _check, _dt, _ptr, _stream, lib

_SM_COUNT = {}


_plans = {}
_plan_epoch = [0]          # bumped when a switch that changes the plans is thrown


def sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def supported(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> bool:
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or a.stride(1) != 1:
        return False
    M, K = a.shape
    ld = a.stride(0)
    # what infero_gemm_tc_supported checks, without the call: it is asked before every product
    return (M > 0 and w.shape[0] > 0 and K >= 8 and K % 8 == 0 and ld % 8 == 0 and ld >= K
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def plan(M: int, N: int, K: int, device) -> Tuple[int, int, int]:
    """(splits, k-tiles per split, workspace bytes) of the few-row path."""
    key = (M, N, K, _plan_epoch[0])
    hit = _plans.get(key)
    if hit is None:
        s, per, ws = c_int(0), c_int(0), c_longlong(0)
        lib().infero_gemm_tc_plan(c_int(M), c_int(N), c_int(K), c_int(sm_count(device)), byref(s), byref(per), byref(ws))
        hit = _plans[key] = (s.value, per.value, ws.value)
    return hit


def gemm(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
         tile_n: int = 0) -> None:
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and out.stride(1) == 1
    ws = None
    ws_bytes = 0
    if M <= 256:
        _, _, ws_bytes = plan(M, N, K, a.device)
        if ws_bytes:
            ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device=a.device)
    _check(lib().infero_gemm_tc(_ptr(a), _ptr(w), _ptr(bias), c_int(_dt(bias) if bias is not None else F32),
                                _ptr(out), c_int(_dt(out)), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
                                c_int(out.stride(0)), _ptr(ws), c_longlong(ws_bytes), c_int(sm_count(a.device)),
                                c_int(tile_n), _stream()))


def set_cluster(on: bool) -> None:
    """Few-row products whose K is cut into splits: add the splits up inside the kernel (a cluster
    per tile, through distributed shared memory) or return them as partial sums (the default;
    ``INFERO_GEMM_CLUSTER=1`` turns the cluster on)."""
    lib().infero_gemm_set_cluster(c_int(1 if on else 0))
    _plan_epoch[0] += 1


def set_pairs(on: bool) -> None:
    """Many-token products on pairs of CTAs (cta_group::2) or on single CTAs; on unless
    ``INFERO_GEMM_PAIR=0``."""
    lib().infero_gemm_set_pairs(c_int(1 if on else 0))


def gemm_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """out[M, N/2] = silu(g) * u where (g_j, u_j) are columns (2j, 2j+1) of a @ w^T.  Returns False
    (nothing launched) when few rows would need more than one split of K."""
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N // 2) and out.stride(1) == 1 and out.dtype == torch.bfloat16
    rc = lib().infero_gemm_tc_swiglu(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
                                     c_int(out.stride(0)), c_int(sm_count(a.device)), _stream())
    if rc == 2:
        return False
    _check(rc)
    return True


def partials(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """float32 [splits, M, N] whose sum over the first axis is a @ w^T (M <= 256)."""
    M, K = a.shape
    N = w.shape[0]
    s, per, _ = plan(M, N, K, a.device)
    if 2 <= s <= 8 and lib().infero_gemm_cluster_enabled():
        # the splits of a tile add up inside the kernel (a cluster per tile): one array comes back
        out = torch.empty((1, M, N), dtype=torch.float32, device=a.device)
        _check(lib().infero_gemm_tc_summed(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                                           c_int(a.stride(0)), c_int(s), c_int(per), _stream()))
        return out
    out = torch.empty((s, M, N), dtype=torch.float32, device=a.device)
    _check(lib().infero_gemm_tc_partials(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                                         c_int(a.stride(0)), c_int(s), c_int(per), _stream()))
    return out


def residual_norm(a: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, bias: Optional[torch.Tensor],
                  norm_w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """A few-row product that is a residual update, with what the RMSNorm behind it needs:
    resid += a @ w^T (+ bias) in place (float32 [M, N]); returns (h, sumsq) with h = bf16(resid * norm_w)
    and sumsq[tile, t] the sum of resid[t, n]^2 over the 128 features n of tile (float32 [tiles, 256]).
    The norm's scalar for token t is rsqrt(sumsq[:, t].sum() / N + eps); ``gemm_swiglu_scaled`` and the
    fused decode attention apply it after their own products."""
    from ctypes import c_float  # noqa: F401
    M, K = a.shape
    N = w.shape[0]
    assert M <= 256 and resid.shape == (M, N) and resid.dtype == torch.float32 and resid.is_contiguous()
    s, per = c_int(0), c_int(0)
    lib().infero_gemm_tc_plan_cluster(c_int(M), c_int(N), c_int(K), c_int(sm_count(a.device)), byref(s), byref(per))
    h = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    sumsq = torch.zeros(((N + 127) // 128, 256), dtype=torch.float32, device=a.device)
    _check(lib().infero_gemm_tc_residual_norm(_ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), s, per,
                                              _ptr(resid), _ptr(bias), c_int(_dt(bias) if bias is not None else F32),
                                              _ptr(norm_w), c_int(_dt(norm_w)), _ptr(h), _ptr(sumsq), _stream()))
    return h, sumsq


def gemm_swiglu_scaled(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, sumsq: torch.Tensor, eps: float) -> bool:
    """``gemm_swiglu`` on an input that lacks its norm's scalar: token t's products are multiplied by
    rsqrt(sumsq[:, t].sum() / K + eps) before the activation.  Few rows, one split of K; else False."""
    from ctypes import c_float
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N // 2) and out.stride(1) == 1 and out.dtype == torch.bfloat16
    assert sumsq.dtype == torch.float32 and sumsq.shape[1] == 256 and sumsq.is_contiguous()
    rc = lib().infero_gemm_tc_swiglu_scaled(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
                                            c_int(out.stride(0)), _ptr(sumsq), c_int(sumsq.shape[0]), c_float(1.0 / K),
                                            c_float(eps), c_int(sm_count(a.device)), _stream())
    if rc == 2:
        return False
    _check(rc)
    return True


def reduce_partials(partial: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    S, M, N = partial.shape
    assert partial.is_contiguous() and partial.dtype == torch.float32 and out.shape == (M, N)
    _check(lib().infero_reduce_partials(_ptr(partial), c_int(S), _ptr(bias),
                                        c_int(_dt(bias) if bias is not None else F32), _ptr(out), c_int(_dt(out)),
                                        c_int(M), c_int(N), c_int(out.stride(0)), _stream()))


def error_flag() -> int:
    """Synchronises; non-zero if a kernel gave up on one of its bounded waits since the flag was last
    read (reading clears it).  1-3: a product kernel, 4: decode attention, 5-7: prompt attention,
    8: the many-row norm."""
    return int(lib().infero_tc_error_flag())


def clear_error_flag() -> None:
    error_flag()


def set_error_flag(value: int) -> None:
    """Write the flag from the host: how tests exercise what the engine does after a wait ran out,
    without any kernel missing one."""
    if lib().infero_tc_set_error_flag(c_int(int(value))):
        raise RuntimeError("cannot write the device's fault flag")
