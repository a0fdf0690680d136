"""The no-allocation decode attention entry point against the ordinary one.

Some embedders of the library cannot call cudaMalloc (all device memory is handed out by
their own start-up code, or a late allocation could stall or fail), so
``infero_attn_decode_static`` keeps the scratch for its context splits in a fixed array
inside the library.  This test calls it through its exported C symbol, twice in a row (the
second call finds the first one's leftovers in the shared array), and compares each result
with what ``infero_attn_decode`` gives with scratch from the caller, and both with a float64
statement of the same attention over the same pages.  It is collected last
so that a run that stops at the first failure has already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, n_tok, H, Hkv, D, lengths, page=16):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-L // page) for L in lengths) + 3
    perm = torch.randperm(pages, generator=g)
    width = max(-(-L // page) for L in lengths) + 1
    table = torch.full((n_tok, width), -1, dtype=torch.int32)
    kc = (torch.randn((pages, Hkv, page, D), generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn((pages, Hkv, page, D), generator=g) * 0.5).to(torch.bfloat16)
    nxt = 0
    for e, L in enumerate(lengths):
        for b in range(-(-L // page)):
            table[e, b] = int(perm[nxt])
            nxt += 1
    q = (torch.randn((n_tok, H * D), generator=g) * 0.5).to(torch.bfloat16)
    positions = torch.tensor([L - 1 for L in lengths], dtype=torch.int32)
    entry = torch.arange(n_tok, dtype=torch.int32)
    return [t.to(DEV) for t in (q, kc, vc, table, entry, positions)]


def _reference(q, kc, vc, table, positions, H, Hkv, D, window, page=16):
    """softmax(q K^T / sqrt(D)) V per token and head in float64, keys gathered through the block
    table: key j is seen from position p iff j <= p and (no window or p - j < window)."""
    q, kc, vc = q.double().cpu(), kc.double().cpu(), vc.double().cpu()
    table, positions = table.cpu(), positions.cpu()
    n_tok, g = q.shape[0], H // Hkv
    out = torch.zeros((n_tok, H, D), dtype=torch.float64)
    for t in range(n_tok):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        js = torch.arange(lo, p + 1)
        pages = table[t, js // page].long()
        for h in range(H):
            keys = kc[pages, h // g, js % page]               # [n, D]
            vals = vc[pages, h // g, js % page]
            w = torch.softmax(keys @ q[t, h * D:(h + 1) * D] / math.sqrt(D), dim=0)
            out[t, h] = w @ vals
    return out.reshape(n_tok, H * D).numpy()


def _args(q, out, kc, vc, table, entry, positions, n_tok, H, Hkv, D, page, window, chunk, splits):
    return [c_void_p(q.data_ptr()), c_int(q.stride(0)), c_void_p(out.data_ptr()), c_int(out.stride(0)),
            c_void_p(kc.data_ptr()), c_void_p(vc.data_ptr()), c_void_p(table.data_ptr()), c_int(table.shape[1]),
            c_void_p(entry.data_ptr()), c_void_p(positions.data_ptr()), c_int(0), c_int(n_tok), c_int(H),
            c_int(Hkv), c_int(D), c_int(page), c_int(window), c_float(1.0 / math.sqrt(D)), c_int(chunk),
            c_int(splits)]


def test_static_scratch_decode_matches_the_allocating_entry_point():
    from infero_b200 import kernels as K
    lib = K.lib()
    static = lib.infero_attn_decode_static            # the exported C symbol itself
    plain = lib.infero_attn_decode
    need = lib.infero_attn_decode_scratch
    need.restype = ctypes.c_longlong
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    shapes = [
        # tokens, heads, kv heads, head size, cached lengths, window, keys per split, splits
        (3, 14, 2, 64, [300, 17, 129], 0, 64, 5),
        (2, 6, 3, 48, [90, 200], 40, 16, 4),           # fewer bytes than the first call left behind
    ]
    for seed, (n_tok, H, Hkv, D, lengths, window, chunk, splits) in enumerate(shapes):
        q, kc, vc, table, entry, positions = _case(seed, n_tok, H, Hkv, D, lengths)
        out_static = torch.zeros((n_tok, H * D), dtype=torch.bfloat16, device=DEV)
        out_plain = torch.zeros_like(out_static)
        a = _args(q, out_static, kc, vc, table, entry, positions, n_tok, H, Hkv, D, 16, window, chunk, splits)
        rc = static(*a, stream)
        assert rc == 0, lib.infero_last_error().decode()
        scratch = torch.empty(int(need(c_int(n_tok), c_int(H), c_int(D), c_int(splits))) // 4,
                              dtype=torch.float32, device=DEV)
        a[2] = c_void_p(out_plain.data_ptr())
        rc = plain(*a, c_void_p(scratch.data_ptr()), stream)
        assert rc == 0, lib.infero_last_error().decode()
        torch.cuda.synchronize()
        got, ref = out_static.float().cpu().numpy(), out_plain.float().cpu().numpy()
        assert np.isfinite(got).all()
        worst = float(np.abs(got - ref).max() / np.abs(ref).max())
        assert worst <= 1.5e-2, f"call {seed}: relative difference {worst:.3e}"   # the kernel tests' bf16 bound
        assert np.abs(ref).max() > 0
        exact = _reference(q, kc, vc, table, positions, H, Hkv, D, window)
        for name, arr in (("the static entry point", got), ("the allocating entry point", ref)):
            worst = float(np.abs(arr - exact).max() / np.abs(exact).max())
            assert worst <= 1.5e-2, f"call {seed}: {name} is {worst:.3e} from the float64 statement"


def test_static_scratch_refuses_what_does_not_fit():
    from infero_b200 import kernels as K
    lib = K.lib()
    n_tok, H, Hkv, D = 64, 64, 8, 128
    q, kc, vc, table, entry, positions = _case(5, 2, 4, 2, 16, [20, 30])
    out = torch.zeros((2, 64), dtype=torch.bfloat16, device=DEV)
    a = _args(q, out, kc, vc, table, entry, positions, n_tok, H, Hkv, D, 16, 0, 64, 16)   # 34 MiB of partials
    rc = lib.infero_attn_decode_static(*a, c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    assert "fixed" in lib.infero_last_error().decode()
    torch.cuda.synchronize()
