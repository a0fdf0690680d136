"""Each CUDA kernel alone against a plain PyTorch float32/float64 statement of the same op,
at sizes other than the engine's tiny configurations."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * scale).to(dtype).to(DEV)


# ---- matrix products ---------------------------------------------------------------------------
def _gemm_ref(a, w, bias):
    out = a.double().cpu() @ w.double().cpu().T
    if bias is not None:
        out += bias.double().cpu()
    return out


def _rel_err(got, ref):
    return float((got.double().cpu() - ref).abs().max() / (ref.abs().max() + 1e-30))


GEMM_TC_SHAPES = [
    # M, N, K  (few rows: weights on the wide side, K in splits; many rows: tokens on the wide side)
    (1, 128, 64), (1, 3584, 3584), (8, 4608, 3584), (8, 3584, 18944), (3, 1000, 96), (16, 777, 224),
    (17, 512, 64), (33, 300, 176), (64, 1152, 896), (65, 2048, 1024), (130, 640, 520), (256, 384, 200),
    (257, 512, 128), (300, 777, 224), (512, 1000, 96), (1024, 4608, 3584), (2048, 1280, 4864), (384, 96, 256),
    (2048, 3584, 320), (1500, 3000, 136), (20000, 200, 72), (511, 130, 64), (769, 3584, 136), (1000, 48, 512),     # tile widths other than 256; many rounds per CTA
]


@pytest.fixture(params=["pairs", "single"])
def cta_pairs(request):
    """Many-token products both ways: on pairs of CTAs sharing an MMA, and on single CTAs."""
    from infero_b200.kernels import tc_gemm
    tc_gemm.set_pairs(request.param == "pairs")
    yield request.param
    tc_gemm.set_pairs(True)


@pytest.mark.parametrize("M,N,K", GEMM_TC_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tensor_core(M, N, K, out_dtype, cta_pairs):
    from infero_b200.kernels import tc_gemm
    if cta_pairs == "single" and M <= 256:
        pytest.skip("few rows take another kernel either way")
    a = _rand((M, K), torch.bfloat16, 1)
    w = _rand((N, K), torch.bfloat16, 2, 0.05)
    bias = _rand((N,), torch.bfloat16, 3)
    assert tc_gemm.supported(a, w)
    for b in (None, bias):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        tc_gemm.gemm(a, w, b, out)
        assert tc_gemm.error_flag() == 0
        err = _rel_err(out, _gemm_ref(a, w, b))
        tol = 1e-5 if out_dtype == torch.float32 else 6e-3       # bf16 output rounds to 2^-9
        assert err <= tol, f"M={M} N={N} K={K} bias={b is not None}: {err:.3e}"


@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_tensor_core_tiles_and_strides(tile_n):
    from infero_b200.kernels import tc_gemm
    M, N, K = 700, 900, 1096
    big = _rand((M, K + 40), torch.bfloat16, 4)
    a = big[:, 8:8 + K]                                 # a strided view: rows 16-byte aligned, stride K + 40
    w = _rand((N, K), torch.bfloat16, 5, 0.05)
    out_big = torch.zeros((M, N + 24), dtype=torch.bfloat16, device=DEV)
    out = out_big[:, :N]
    assert tc_gemm.supported(a, w)
    tc_gemm.gemm(a, w, None, out, tile_n=tile_n)
    assert tc_gemm.error_flag() == 0
    assert _rel_err(out, _gemm_ref(a, w, None)) <= 6e-3
    assert float(out_big[:, N:].abs().max()) == 0.0, "wrote outside its columns"


def test_gemm_tensor_core_partials_sum_in_fixed_order():
    from infero_b200.kernels import tc_gemm
    M, N, K = 8, 3584, 18944
    a = _rand((M, K), torch.bfloat16, 6)
    w = _rand((N, K), torch.bfloat16, 7, 0.02)
    p1 = tc_gemm.partials(a, w)
    p2 = tc_gemm.partials(a, w)
    assert p1.shape[0] > 1, "this shape was meant to be cut along K"
    assert torch.equal(p1, p2)
    out = torch.empty((M, N), dtype=torch.float32, device=DEV)
    tc_gemm.reduce_partials(p1, None, out)
    assert _rel_err(out, _gemm_ref(a, w, None)) <= 1e-5
    assert tc_gemm.error_flag() == 0


@pytest.mark.parametrize("M,N,K", [(8, 3584, 18944), (64, 4608, 3584), (1, 3584, 3584), (200, 1000, 2048), (33, 130, 1024),
                                   (256, 896, 4864)])
def test_gemm_tensor_core_splits_added_inside_a_cluster(M, N, K):
    """The splits of a tile as one cluster, added up through distributed shared memory: the same
    sums in the same order as the partial sums added up afterwards, bit for bit."""
    import ctypes
    from infero_b200.kernels import tc_gemm
    a = _rand((M, K), torch.bfloat16, 8)
    w = _rand((N, K), torch.bfloat16, 9, 0.02)
    tc_gemm.set_cluster(True)
    try:
        s, per, _ = tc_gemm.plan(M, N, K, DEV)
        assert 2 <= s <= 8, "this shape was meant to be cut along K"
        summed = tc_gemm.partials(a, w)
        assert summed.shape == (1, M, N)
        again = tc_gemm.partials(a, w)
        assert torch.equal(summed, again)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
        tc_gemm.gemm(a, w, None, out)                      # the whole product through the same kernel
        assert _rel_err(out, _gemm_ref(a, w, None)) <= 6e-3
    finally:
        tc_gemm.set_cluster(False)
    parts = torch.full((s, M, N), float("nan"), dtype=torch.float32, device=DEV)
    L = tc_gemm.lib()
    rc = L.infero_gemm_tc_partials(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                                   ctypes.c_void_p(parts.data_ptr()), M, N, K, a.stride(0), s, per,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    ref = torch.empty((M, N), dtype=torch.float32, device=DEV)
    tc_gemm.reduce_partials(parts, None, ref)
    assert torch.equal(summed[0], ref)
    assert _rel_err(ref, _gemm_ref(a, w, None)) <= 1e-5
    assert tc_gemm.error_flag() == 0


@pytest.mark.parametrize("M,N,K", [(8, 37888, 3584), (64, 1024, 512), (300, 400, 264), (2048, 1280, 512), (5, 354, 64),
                                   (2048, 7168, 192), (700, 3000, 72)])
def test_gemm_tensor_core_with_swiglu_epilogue(M, N, K, cta_pairs):
    from infero_b200.kernels import tc_gemm
    if cta_pairs == "single" and M <= 256:
        pytest.skip("few rows take another kernel either way")
    a = _rand((M, K), torch.bfloat16, 1)
    w = _rand((N, K), torch.bfloat16, 2, 0.1)
    out = torch.full((M, N // 2), 7.0, dtype=torch.bfloat16, device=DEV)
    if not tc_gemm.gemm_swiglu(a, w, out):
        splits, _, _ = tc_gemm.plan(M, N, K, DEV)
        assert M <= 256 and splits > 1
        return
    y = a.double() @ w.double().T
    g, u = y[:, 0::2], y[:, 1::2]
    ref = g / (1 + torch.exp(-g)) * u
    assert float((out.double() - ref).abs().max() / ref.abs().max()) <= 6e-3
    assert tc_gemm.error_flag() == 0


@pytest.mark.parametrize("M,N,K", [(8, 3584, 18944), (1, 3584, 3584), (64, 896, 4864), (200, 1000, 2048), (5, 128, 320),
                                   (16, 256, 616), (33, 130, 1024)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_product_that_updates_the_residual_and_prepares_the_norm(M, N, K, with_bias):
    """resid += a w^T (+ bias); h = bf16(resid * norm_w); per-tile sums of squares -- against float64,
    and the norm that follows from (h, sums) against the norm computed in one piece."""
    from infero_b200.kernels import tc_gemm
    a = _rand((M, K), torch.bfloat16, 1)
    w = _rand((N, K), torch.bfloat16, 2, scale=1.0 / math.sqrt(K))
    bias = _rand((N,), torch.float32, 3) if with_bias else None
    norm_w = (1.0 + _rand((N,), torch.float32, 4, scale=0.1))
    resid0 = _rand((M, N), torch.float32, 5, scale=2.0)
    resid = resid0.clone()
    h, sumsq = tc_gemm.residual_norm(a, w, resid, bias, norm_w)
    torch.cuda.synchronize()
    ref = resid0.double() + a.double() @ w.double().T + (bias.double() if with_bias else 0)
    assert _rel_err(resid, ref.cpu()) <= 2e-5
    assert _rel_err(h.float(), (ref * norm_w.double()).cpu()) <= 5e-3                    # one bf16 rounding
    tiles = (N + 127) // 128
    pad = torch.zeros((M, tiles * 128), dtype=torch.float64, device=DEV)
    pad[:, :N] = ref
    ss_ref = (pad.view(M, tiles, 128) ** 2).sum(-1).T                            # [tiles, M]
    assert _rel_err(sumsq[:, :M], ss_ref.cpu()) <= 2e-5
    eps = 1e-6
    rstd = torch.rsqrt(sumsq[:, :M].double().sum(0) / N + eps)
    normed_ref = ref * torch.rsqrt((ref ** 2).mean(-1, keepdim=True) + eps) * norm_w.double()
    assert _rel_err(h.double() * rstd[:, None], normed_ref.cpu()) <= 5e-3
    assert tc_gemm.error_flag() == 0


@pytest.mark.parametrize("M,N,K", [(8, 37888, 3584), (1, 1232, 256), (64, 1024, 512), (5, 640, 128), (130, 354, 64)])
def test_swiglu_product_that_applies_the_norms_scalar(M, N, K):
    from infero_b200.kernels import tc_gemm
    a = _rand((M, K), torch.bfloat16, 1)
    w = _rand((N, K), torch.bfloat16, 2, scale=1.0 / math.sqrt(K))
    tiles = (K + 127) // 128
    sumsq = torch.rand((tiles, 256), generator=torch.Generator().manual_seed(3)).to(DEV) * 50.0
    eps = 1e-5
    out = torch.zeros((M, N // 2), dtype=torch.bfloat16, device=DEV)
    if not tc_gemm.gemm_swiglu_scaled(a, w, out, sumsq, eps):
        pytest.skip("this shape cuts K into splits: the scaled epilogue is not used for it")
    rstd = torch.rsqrt(sumsq[:, :M].double().sum(0) / K + eps)
    y = (a.double() @ w.double().T) * rstd[:, None]
    g, u = y[:, 0::2], y[:, 1::2]
    ref = g / (1 + torch.exp(-g)) * u
    assert _rel_err(out.float(), ref.cpu()) <= 1e-2
    assert tc_gemm.error_flag() == 0


def test_gemm_tensor_core_refuses_what_it_cannot_take():
    from infero_b200.kernels import tc_gemm
    a = _rand((4, 100), torch.bfloat16, 1)               # K = 100 is no multiple of 8
    w = _rand((32, 100), torch.bfloat16, 2)
    assert not tc_gemm.supported(a, w)
    a = _rand((4, 104), torch.bfloat16, 1)[:, 1:97]      # misaligned start
    assert not tc_gemm.supported(a, _rand((32, 96), torch.bfloat16, 2))


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (5, 130, 67), (70, 65, 129), (3, 1000, 96)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_gemm_tiled(M, N, K, dt):
    from infero_b200 import kernels as Kn
    a, w, bias = _rand((M, K), dt, 1), _rand((N, K), dt, 2, 0.1), _rand((N,), dt, 3)
    out = torch.empty((M, N), dtype=torch.float32, device=DEV)
    Kn.gemm_tiled(a, w, bias, out)
    assert _rel_err(out, _gemm_ref(a, w, bias)) <= 2e-6


def test_gemm_tiled_rows_do_not_depend_on_the_batch():
    from infero_b200 import kernels as Kn
    a, w = _rand((77, 200), torch.float32, 1), _rand((90, 200), torch.float32, 2)
    full = torch.empty((77, 90), dtype=torch.float32, device=DEV)
    Kn.gemm_tiled(a, w, None, full)
    for rows in ([5], [0, 76], list(range(60, 70))):
        sub = a[rows].contiguous()
        out = torch.empty((len(rows), 90), dtype=torch.float32, device=DEV)
        Kn.gemm_tiled(sub, w, None, out)
        assert torch.equal(out, full[rows])


@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_gemm_skinny(M):
    from infero_b200 import kernels as Kn
    N, K = 1003, 520
    a, w, bias = _rand((M, K), torch.bfloat16, 1), _rand((N, K), torch.bfloat16, 2, 0.1), _rand((N,), torch.float32, 3)
    out = torch.empty((M, N), dtype=torch.float32, device=DEV)
    Kn.gemm_skinny(a, w, bias, out)
    assert _rel_err(out, _gemm_ref(a, w, bias)) <= 1e-5


# ---- embedding, norm, activation ---------------------------------------------------------------
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_embed_gather(dt):
    from infero_b200 import kernels as Kn
    table = _rand((301, 136), dt, 1)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    x = torch.empty((5, 136), dtype=torch.float32, device=DEV)
    Kn.embed_gather(table, ids, x, 1.0)
    assert torch.equal(x, table[ids.long()].float())


@pytest.mark.parametrize("d", [40, 1000, 3584])
@pytest.mark.parametrize("eps", [1e-6, 1e-3])
@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(d, eps, act):
    from infero_b200 import kernels as Kn
    T = 7
    x = _rand((T, d), torch.float32, 1)
    delta = _rand((T, d), act, 2)
    w = _rand((d,), act, 3) + 1
    x0 = x.clone()
    out = torch.empty((T, d), dtype=act, device=DEV)
    Kn.add_rmsnorm(x, delta, w, eps, out)
    v = x0.double() + delta.double()
    ref = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w.double()
    assert torch.allclose(x.double(), v.float().double(), atol=0, rtol=0)
    tol = 1e-6 if act == torch.float32 else 5e-3
    assert float((out.double() - ref).abs().max() / ref.abs().max()) <= tol
    # selected rows, no write-back
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    x1 = x0.clone()
    out2 = torch.empty((3, d), dtype=act, device=DEV)
    Kn.add_rmsnorm(x1, delta, w, eps, out2, rows)
    assert torch.equal(x1, x0)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [96, 100, 3584, 5120])
@pytest.mark.parametrize("T", [300, 3000])
def test_add_rmsnorm_many_rows_equal_few_rows_bit_for_bit(act, d, T):
    """Many rows at once (the kernels that keep several rows on their way: through a ring in shared
    memory where a row is a multiple of 16 bytes, from registers where it is not, as with 100 bf16
    values; 3,000 rows make every block refill its ring) against the same rows 100 at a time."""
    from infero_b200 import kernels as Kn
    x = _rand((T, d), torch.float32, 1)
    delta = _rand((T, d), act, 2)
    w = _rand((d,), act, 3) + 1
    xa, xb = x.clone(), x.clone()
    oa = torch.empty((T, d), dtype=act, device=DEV)
    ob = torch.empty_like(oa)
    Kn.add_rmsnorm(xa, delta, w, 1e-6, oa)
    for t0 in range(0, T, 100):
        Kn.add_rmsnorm(xb[t0:t0 + 100], delta[t0:t0 + 100], w, 1e-6, ob[t0:t0 + 100])
    assert torch.equal(xa, xb) and torch.equal(oa, ob)
    v = x.double() + delta.double()
    ref = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + 1e-6) * w.double()
    assert float((oa.double() - ref).abs().max() / ref.abs().max()) <= (1e-6 if act == torch.float32 else 5e-3)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_swiglu(dt):
    from infero_b200 import kernels as Kn
    T, ff = 5, 333
    gu = _rand((T, 2 * ff), dt, 1, 3.0)
    out = torch.empty((T, ff), dtype=dt, device=DEV)
    Kn.swiglu(gu, out)
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()
    ref = g / (1 + torch.exp(-g)) * u
    tol = 1e-6 if dt == torch.float32 else 5e-3
    assert float((out.double() - ref).abs().max() / ref.abs().max()) <= tol


# ---- rotary + cache append, attention ----------------------------------------------------------
def _rope_ref(x, pos, theta, rotary):
    half = rotary // 2
    inv = theta ** (-2.0 * torch.arange(half, dtype=torch.float64) / rotary)
    ang = pos.double()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:rotary]
    out[..., :half] = a * c - b * s
    out[..., half:rotary] = a * s + b * c
    return out


@pytest.mark.parametrize("H,Hkv,D,rotary", [(6, 3, 48, 48), (5, 5, 80, 40), (7, 1, 128, 128)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rope_and_cache_append(H, Hkv, D, rotary, dt):
    from infero_b200 import kernels as Kn
    P, pages, T = 16, 12, 9
    theta = 50000.0
    qkv = _rand((T, (H + 2 * Hkv) * D), dt, 1)
    qkv0 = qkv.clone()
    # two requests: entry 0 at positions 30..34 (pages 1 and 2 of its table), entry 1 at 0..3
    positions = torch.tensor([30, 31, 32, 33, 34, 0, 1, 2, 3], dtype=torch.int32, device=DEV)
    entry = torch.tensor([0] * 5 + [1] * 4, dtype=torch.int32, device=DEV)
    table = torch.tensor([[7, 3, 9, -1], [11, -1, -1, -1]], dtype=torch.int32, device=DEV)
    kc = torch.zeros((pages, Hkv, P, D), dtype=dt, device=DEV)
    vc = torch.zeros_like(kc)
    half = rotary // 2
    inv = torch.from_numpy((np.float64(theta) ** (-2.0 * np.arange(half) / rotary)).astype(np.float32)).to(DEV)
    Kn.rope_cache(qkv, positions, entry, table, inv, kc, vc, H, Hkv, D, P)
    q0 = qkv0[:, :H * D].double().cpu().view(T, H, D)
    k0 = qkv0[:, H * D:(H + Hkv) * D].double().cpu().view(T, Hkv, D)
    v0 = qkv0[:, (H + Hkv) * D:].cpu().view(T, Hkv, D)
    qr, kr = _rope_ref(q0, positions.cpu(), theta, rotary), _rope_ref(k0, positions.cpu(), theta, rotary)
    tol = 2e-6 if dt == torch.float32 else 8e-3
    assert float((qkv[:, :H * D].double().cpu().view(T, H, D) - qr).abs().max()) <= tol * float(qr.abs().max())
    tb = table.cpu()
    for t in range(T):
        p, e = int(positions[t]), int(entry[t])
        page, row = int(tb[e, p // P]), p % P
        assert float((kc[page, :, row].double().cpu() - kr[t]).abs().max()) <= tol * float(kr.abs().max())
        assert torch.equal(vc[page, :, row].cpu(), v0[t])
    assert int((kc != 0).any(-1).sum()) == T * Hkv, "keys were written to rows that belong to no token"


@pytest.mark.parametrize("H,Hkv,D,rotary", [(6, 3, 48, 48), (5, 5, 80, 48), (28, 4, 128, 128)])
def test_rope_and_cache_append_many_tokens(H, Hkv, D, rotary):
    """The one-block-per-token kernel (16 tokens and more, bf16) gives bit for bit what the
    per-head kernel gives on the same tokens, eight at a time."""
    from infero_b200 import kernels as Kn
    P, pages, T = 16, 16, 45
    dt = torch.bfloat16
    qkv = _rand((T, (H + 2 * Hkv) * D), dt, 1)
    positions = torch.tensor(list(range(20, 50)) + list(range(0, 15)), dtype=torch.int32, device=DEV)
    entry = torch.tensor([0] * 30 + [1] * 15, dtype=torch.int32, device=DEV)
    table = torch.tensor([[7, 3, 9, 12], [11, -1, -1, -1]], dtype=torch.int32, device=DEV)
    inv = torch.from_numpy((np.float64(1e4) ** (-2.0 * np.arange(rotary // 2) / rotary)).astype(np.float32)).to(DEV)
    a, b = qkv.clone(), qkv.clone()
    kc1 = torch.zeros((pages, Hkv, P, D), dtype=dt, device=DEV); vc1 = torch.zeros_like(kc1)
    kc2 = torch.zeros_like(kc1); vc2 = torch.zeros_like(kc1)
    Kn.rope_cache(a, positions, entry, table, inv, kc1, vc1, H, Hkv, D, P)
    for t0 in range(0, T, 8):
        Kn.rope_cache(b[t0:t0 + 8], positions[t0:t0 + 8].contiguous(), entry[t0:t0 + 8].contiguous(), table, inv,
                      kc2, vc2, H, Hkv, D, P)
    assert torch.equal(a, b) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert int((kc1 != 0).any(-1).sum()) == T * Hkv


def _attention_ref(q, keys, values, scale, window):
    """q [H, D] at the last position of keys [L, Hkv, D]."""
    H, D = q.shape
    L, Hkv, _ = keys.shape
    g = H // Hkv
    lo = max(0, L - window) if window else 0
    out = torch.zeros(H, D, dtype=torch.float64)
    for h in range(H):
        s = (keys[lo:, h // g] @ q[h]) * scale
        p = torch.softmax(s, dim=0)
        out[h] = p @ values[lo:, h // g]
    return out


@pytest.mark.parametrize("H,Hkv,D", [(6, 3, 48), (7, 1, 128), (4, 4, 80), (10, 2, 64)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 40])
def test_attention_over_pages(H, Hkv, D, dt, window):
    """Mixed batch: a long prompt portion, a decode token far into its request, a fresh request.
    One key per request gets a large score so that a lost or misplaced key shows."""
    from infero_b200 import kernels as Kn
    from infero_b200.kernels import attention as A
    P, pages = 16, 40
    lens = [(0, 70), (133, 1), (50, 23), (0, 1)]          # (tokens already cached, new tokens)
    rng = np.random.default_rng(0)
    perm = rng.permutation(pages)
    table = torch.full((len(lens), 12), -1, dtype=torch.int32)
    nxt = 0
    K_all, V_all = [], []
    kc = torch.zeros((pages, Hkv, P, D), dtype=dt, device=DEV)
    vc = torch.zeros_like(kc)
    for e, (old, new) in enumerate(lens):
        L = old + new
        k = _rand((L, Hkv, D), dt, 10 + e)
        v = _rand((L, Hkv, D), dt, 20 + e)
        K_all.append(k)
        V_all.append(v)
        for b in range(-(-L // P)):
            table[e, b] = int(perm[nxt]); nxt += 1
            n = min(P, L - b * P)
            kc[table[e, b], :, :n] = k[b * P:b * P + n].transpose(0, 1)
            vc[table[e, b], :, :n] = v[b * P:b * P + n].transpose(0, 1)
    T = sum(n for _, n in lens)
    q = _rand((T, H * D), dt, 3)
    scale = 1.0 / math.sqrt(D)
    # make key 5 of request 0 and key 100 of request 1 stand out for head 0
    q3 = q.view(T, H, D)
    for e, j in ((0, 5), (1, 100)):
        t0 = sum(n for _, n in lens[:e])
        kk = K_all[e][j, 0].float()
        q3[t0:t0 + lens[e][1], 0] = (kk * (6.0 / scale / float(kk @ kk))).to(dt)
    positions = torch.tensor([old + i for old, n in lens for i in range(n)], dtype=torch.int32, device=DEV)
    entry = torch.tensor([e for e, (_, n) in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    out = torch.empty((T, H * D), dtype=dt, device=DEV)
    A.attention_any(q, out, kc, vc, table.to(DEV), entry, positions, H, Hkv, D, P, window, scale,
                    q_lens=[n for _, n in lens], pos0=[o for o, _ in lens])
    t = 0
    worst = 0.0
    for e, (old, new) in enumerate(lens):
        for i in range(new):
            L = old + i + 1
            ref = _attention_ref(q3[t].double().cpu(), K_all[e][:L].double().cpu(), V_all[e][:L].double().cpu(),
                                 scale, window)
            got = out[t].double().cpu().view(H, D)
            worst = max(worst, float((got - ref).abs().max() / ref.abs().max()))
            t += 1
    assert worst <= (3e-6 if dt == torch.float32 else 1.5e-2), f"{worst:.3e}"


SMALL_PORTIONS = [(0, 300), (300, 260), (77, 2), (129, 1)]        # 8 blocks of 128 rows
LARGE_PORTIONS = [(0, 700), (300, 500), (77, 2), (129, 1)]        # 12 blocks


@pytest.mark.parametrize("H,Hkv,D,P,lens", [
    (7, 1, 128, 16, SMALL_PORTIONS), (7, 1, 128, 64, SMALL_PORTIONS),
    (4, 2, 64, 16, SMALL_PORTIONS), (4, 2, 64, 64, SMALL_PORTIONS),
    # enough (kv head, pair of heads, block) CTAs to fill the SMs: the kernel then gives a CTA two heads
    (28, 4, 128, 16, LARGE_PORTIONS), (28, 4, 64, 32, LARGE_PORTIONS)])
@pytest.mark.parametrize("window", [None, 200])
def test_prefill_attention_on_tensor_memory(H, Hkv, D, window, P, lens):
    """Prompt portions that span several blocks of 128 rows and several tiles of 128 keys: a
    request from its start, one that continues 300 cached tokens, and a two-token portion; with
    one head per CTA (small grids) and with two."""
    from infero_b200.kernels import attention as A
    dt = torch.bfloat16
    pages = sum(-(-(o + n) // P) for o, n in lens) + 4
    rng = np.random.default_rng(3)
    perm = rng.permutation(pages)
    table = torch.full((len(lens), max(-(-(o + n) // P) for o, n in lens) + 1), -1, dtype=torch.int32)
    kc = _rand((pages, Hkv, P, D), dt, 50)
    vc = _rand((pages, Hkv, P, D), dt, 51)
    Ks, Vs = [], []
    nxt = 0
    for e, (o, n) in enumerate(lens):
        L = o + n
        k, v = _rand((L, Hkv, D), dt, 60 + e), _rand((L, Hkv, D), dt, 80 + e)
        Ks.append(k); Vs.append(v)
        for b in range(-(-L // P)):
            table[e, b] = int(perm[nxt]); nxt += 1
            m = min(P, L - b * P)
            kc[table[e, b], :, :m] = k[b * P:b * P + m].transpose(0, 1)
            vc[table[e, b], :, :m] = v[b * P:b * P + m].transpose(0, 1)
    T = sum(n for _, n in lens)
    scale = 1.0 / math.sqrt(D)
    width = (H + 2 * Hkv) * D                              # q sits in front of a wider row, as in the model
    qkv = _rand((T, width), dt, 7)
    q = qkv[:, :H * D]
    # one far key per request dominates head 0 for its last rows
    t0 = 0
    for e, (o, n) in enumerate(lens):
        j = max(0, o + n - 150) if window else (o + n) // 4
        kk = Ks[e][j, 0].float()
        qkv[t0 + n - 1, :D] = (kk * (6.0 / scale / float(kk @ kk))).to(dt)
        t0 += n
    positions = torch.tensor([o + i for o, n in lens for i in range(n)], dtype=torch.int32, device=DEV)
    entry = torch.tensor([e for e, (_, n) in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    out = torch.zeros((T, H * D), dtype=dt, device=DEV)
    assert A.prefill_tc_supported(q, out, D, P)
    # the first request goes first (no leading single-token request), so everything takes the prefill path
    A.attention_any(q, out, kc, vc, table.to(DEV), entry, positions, H, Hkv, D, P, window, scale,
                    q_lens=[n for _, n in lens], pos0=[o for o, _ in lens])
    worst = 0.0
    bad = []
    t = 0
    for e, (o, n) in enumerate(lens):
        for i in range(n):
            L = o + i + 1
            ref = _attention_ref(qkv[t, :H * D].double().cpu().view(H, D), Ks[e][:L].double().cpu(),
                                 Vs[e][:L].double().cpu(), scale, window)
            got = out[t].double().cpu().view(H, D)
            err = float((got - ref).abs().max() / ref.abs().max())
            if err > 1.5e-2:
                bad.append((e, i, [round(float(x), 3) for x in ((got - ref).abs().amax(dim=1) / ref.abs().max())]))
            worst = max(worst, err)
            t += 1
    assert worst <= 1.5e-2, f"{worst:.3e} at (request, row, per-head error): {bad[:6]} ... {len(bad)} rows"
    from infero_b200.kernels import tc_gemm
    assert tc_gemm.error_flag() == 0


@pytest.mark.parametrize("H,Hkv,D", [(28, 4, 128), (14, 2, 64), (20, 1, 128), (3, 3, 64)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("P", [16, 64])
def test_decode_attention_fed_by_tma(H, Hkv, D, window, P, monkeypatch):
    """Single-token requests of very different lengths (one key, a page edge, hundreds of keys)
    on scattered pages; one far key per request is made to dominate head 0."""
    from infero_b200.kernels import attention as A
    assert A.lib().infero_attn_decode_tma_supported(D, P)
    lengths = [1, 16, 17, 64, 333, 700, 129]
    dt = torch.bfloat16
    n = len(lengths)
    pages = sum(-(-L // P) for L in lengths) + 5
    rng = np.random.default_rng(1)
    perm = rng.permutation(pages)
    table = torch.full((n, max(-(-L // P) for L in lengths) + 2), -1, dtype=torch.int32)
    kc = _rand((pages, Hkv, P, D), dt, 50)               # unused rows hold finite junk, as reused pages do
    vc = _rand((pages, Hkv, P, D), dt, 51)
    Ks, Vs = [], []
    nxt = 0
    for e, L in enumerate(lengths):
        k, v = _rand((L, Hkv, D), dt, 60 + e), _rand((L, Hkv, D), dt, 80 + e)
        Ks.append(k); Vs.append(v)
        for b in range(-(-L // P)):
            table[e, b] = int(perm[nxt]); nxt += 1
            m = min(P, L - b * P)
            kc[table[e, b], :, :m] = k[b * P:b * P + m].transpose(0, 1)
            vc[table[e, b], :, :m] = v[b * P:b * P + m].transpose(0, 1)
    scale = 1.0 / math.sqrt(D)
    q = _rand((n, H * D), dt, 7)
    q3 = q.view(n, H, D)
    for e, L in enumerate(lengths):
        j = max(0, L - 90) if window else L // 3          # inside the window when there is one
        kk = Ks[e][j, 0].float()
        q3[e, 0] = (kk * (6.0 / scale / float(kk @ kk))).to(dt)
    positions = torch.tensor([L - 1 for L in lengths], dtype=torch.int32, device=DEV)
    entry = torch.arange(n, dtype=torch.int32, device=DEV)
    # (bound, arrival counters offered): the plan of a captured step covers more keys than there are;
    # with too few counters for the batch a separate kernel merges the splits
    for bound, counters in ((None, A.N_COUNTERS), (2048, A.N_COUNTERS), (2048, 1)):
        monkeypatch.setattr(A, "N_COUNTERS", counters)
        # the scratch for the splits' partial results comes from the allocator uninitialised: make
        # sure the block it gets is full of NaN, as reused memory may be
        vis = bound or max(lengths)
        if window:
            vis = min(vis, window + 15)
        chunk, splits = A.plan_decode(n, Hkv, H // Hkv, vis)
        poison = torch.full((int(A.lib_scratch(n, H, D, splits)) // 4,), float("nan"), dtype=torch.float32, device=DEV)
        del poison
        out = torch.zeros((n, H * D), dtype=dt, device=DEV)
        A.attention_any(q, out, kc, vc, table.to(DEV), entry, positions, H, Hkv, D, P, window, scale,
                        q_lens=[1] * n, pos0=[L - 1 for L in lengths], kv_bound=bound)
        worst = 0.0
        for e, L in enumerate(lengths):
            ref = _attention_ref(q3[e].double().cpu(), Ks[e].double().cpu(), Vs[e].double().cpu(), scale, window)
            worst = max(worst, float((out[e].double().cpu().view(H, D) - ref).abs().max() / ref.abs().max()))
        assert worst <= 1.5e-2, f"bound {bound}, {counters} counters: {worst:.3e}"
    from infero_b200.kernels import tc_gemm
    assert tc_gemm.error_flag() == 0


@pytest.mark.parametrize("H,Hkv,D,rotary", [(28, 4, 128, 128), (14, 2, 64, 64), (20, 1, 128, 64), (3, 3, 64, 0)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("splits_in", [1, 10])
def test_decode_attention_that_finishes_the_qkv_product_itself(H, Hkv, D, rotary, window, splits_in):
    """The fused launch (bias, rotary positions, cache append, attention from 32-bit partial sums) against
    the two kernels it replaces, bit for bit in the output and in the cache, and against float64."""
    from infero_b200 import kernels as Kn
    from infero_b200.kernels import attention as A, tc_gemm
    P, dt = 16, torch.bfloat16
    lengths = [1, 16, 17, 64, 333, 700, 129, 257]
    n = len(lengths)
    pages = sum(-(-L // P) for L in lengths) + 5
    perm = np.random.default_rng(3).permutation(pages)
    table = torch.full((n, max(-(-L // P) for L in lengths) + 2), -1, dtype=torch.int32)
    kc = _rand((pages, Hkv, P, D), dt, 50)
    vc = _rand((pages, Hkv, P, D), dt, 51)
    Ks, Vs = [], []
    nxt = 0
    for e, L in enumerate(lengths):
        k, v = _rand((L, Hkv, D), dt, 60 + e), _rand((L, Hkv, D), dt, 80 + e)      # the last row is replaced below
        Ks.append(k); Vs.append(v)
        for b in range(-(-L // P)):
            table[e, b] = int(perm[nxt]); nxt += 1
            m = min(P, L - b * P)
            kc[table[e, b], :, :m] = k[b * P:b * P + m].transpose(0, 1)
            vc[table[e, b], :, :m] = v[b * P:b * P + m].transpose(0, 1)
    table = table.to(DEV)
    width = (H + 2 * Hkv) * D
    parts = _rand((splits_in, n, width), torch.float32, 9, scale=1.0 / math.sqrt(splits_in))
    bias = _rand((width,), torch.float32, 10, scale=0.3)
    qkv = Kn.Partials(parts, bias)
    theta = 10000.0
    inv = (theta ** (-torch.arange(0, rotary, 2, dtype=torch.float64) / max(rotary, 1))).to(torch.float32).to(DEV)
    positions = torch.tensor([L - 1 for L in lengths], dtype=torch.int32, device=DEV)
    entry = torch.arange(n, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    vis = min(max(lengths), window + 15) if window else max(lengths)
    for plan in (A.plan_decode(n, Hkv, H // Hkv, vis), (64, -(-vis // 64)), (16, -(-vis // 16))):
        chunk, splits = plan
        if splits > A.MAX_SPLITS:
            continue
        # the two kernels
        k1, v1 = kc.clone(), vc.clone()
        q1 = torch.empty((n, H * D), dtype=dt, device=DEV)
        Kn.rope_cache_partials(qkv, q1, positions, entry, table, inv, k1, v1, H, Hkv, D, P)
        out1 = torch.zeros((n, H * D), dtype=dt, device=DEV)
        A.decode(q1, out1, k1, v1, table, entry, positions, 0, n, H, Hkv, D, P, window, scale, chunk, splits)
        # the one kernel
        k2, v2 = kc.clone(), vc.clone()
        out2 = torch.zeros_like(out1)
        A.decode_fused(qkv, out2, k2, v2, table, entry, positions, inv, H, Hkv, D, P, window, scale, chunk, splits)
        torch.cuda.synchronize()
        assert torch.equal(k1, k2) and torch.equal(v1, v2), f"plan {plan}: the caches differ"
        assert torch.equal(out1, out2), f"plan {plan}: outputs differ by {(out1.float() - out2.float()).abs().max()}"
        # float64: the token's own q, k, v from the summed product, rotated
        full = (parts.double().sum(0) + bias.double()).cpu()
        worst = 0.0
        for e, L in enumerate(lengths):
            row = full[e]
            pos = torch.tensor([L - 1])
            qe = _rope_ref(row[:H * D].view(1, H, D), pos, theta, rotary)[0] if rotary else row[:H * D].view(H, D)
            ke = row[H * D:(H + Hkv) * D].view(1, Hkv, D)
            ke = _rope_ref(ke, pos, theta, rotary)[0] if rotary else ke[0]
            ve = row[(H + Hkv) * D:].view(Hkv, D)
            keys, vals = Ks[e].double().cpu().clone(), Vs[e].double().cpu().clone()
            keys[L - 1], vals[L - 1] = ke, ve
            ref = _attention_ref(qe, keys, vals, scale, window)
            worst = max(worst, float((out2[e].double().cpu().view(H, D) - ref).abs().max() / ref.abs().max()))
        assert worst <= 2e-2, f"plan {plan}: {worst:.3e} from the float64 statement"
    assert tc_gemm.error_flag() == 0


def _paged_requests(totals, Hkv, D, P, dt, seed, dead_before):
    """Keys and values of requests of ``totals`` tokens on scattered pages.  Pages that lie wholly
    before position ``dead_before[e]`` are not held any more (table entry -1), as after the cache
    manager has taken back what a window passed.  Unused rows hold finite junk, as reused pages do."""
    pages = sum(-(-L // P) for L in totals) + 5
    rng = np.random.default_rng(seed)
    perm = rng.permutation(pages)
    table = torch.full((len(totals), max(-(-L // P) for L in totals) + 2), -1, dtype=torch.int32)
    kc, vc = _rand((pages, Hkv, P, D), dt, 50 + seed), _rand((pages, Hkv, P, D), dt, 51 + seed)
    Ks, Vs, nxt = [], [], 0
    for e, L in enumerate(totals):
        k, v = _rand((L, Hkv, D), dt, 60 + e), _rand((L, Hkv, D), dt, 80 + e)
        Ks.append(k); Vs.append(v)
        for b in range(-(-L // P)):
            page = int(perm[nxt]); nxt += 1
            m = min(P, L - b * P)
            kc[page, :, :m] = k[b * P:b * P + m].transpose(0, 1)
            vc[page, :, :m] = v[b * P:b * P + m].transpose(0, 1)
            if b * P + P - 1 >= dead_before[e]:
                table[e, b] = page
    return table, kc, vc, Ks, Vs


@pytest.mark.parametrize("H,Hkv,D", [(4, 2, 64), (7, 1, 128)])
@pytest.mark.parametrize("window", [48, 100])
@pytest.mark.parametrize("P", [16, 64])
def test_window_edge_in_decode_attention_fed_by_tma(H, Hkv, D, window, P):
    """The edge of the window, to the key.  From position p the keys p - W + 1 .. p are seen.  Requests
    come in pairs of equal length: in the first of a pair key p - W + 1 (the oldest one inside) is given
    a score that dominates head 0, so losing it shows; in the second key p - W (the youngest one
    outside) gets that score, so seeing it shows.  Pages the window has passed are not held (-1)."""
    from infero_b200.kernels import attention as A
    assert A.lib().infero_attn_decode_tma_supported(D, P)
    dt = torch.bfloat16
    lengths = [L for L in (window + 1, window + 2, 129, 333, 700) for _ in (0, 1)]
    n = len(lengths)
    table, kc, vc, Ks, Vs = _paged_requests(lengths, Hkv, D, P, dt, 1, [L - window for L in lengths])
    assert int((table == -1).sum(1).max()) > 2
    scale = 1.0 / math.sqrt(D)
    q = _rand((n, H * D), dt, 7)
    q3 = q.view(n, H, D)
    for e, L in enumerate(lengths):
        p = L - 1
        j = p - window + 1 if e % 2 == 0 else p - window
        kk = Ks[e][j, 0].float()
        q3[e, 0] = (kk * (7.0 / scale / float(kk @ kk))).to(dt)
    positions = torch.tensor([L - 1 for L in lengths], dtype=torch.int32, device=DEV)
    entry = torch.arange(n, dtype=torch.int32, device=DEV)
    out = torch.zeros((n, H * D), dtype=dt, device=DEV)
    A.attention_any(q, out, kc, vc, table.to(DEV), entry, positions, H, Hkv, D, P, window, scale,
                    q_lens=[1] * n, pos0=[L - 1 for L in lengths])
    for e, L in enumerate(lengths):
        ref = _attention_ref(q3[e].double().cpu(), Ks[e].double().cpu(), Vs[e].double().cpu(), scale, window)
        err = float((out[e].double().cpu().view(H, D) - ref).abs().max() / ref.abs().max())
        what = "the oldest key inside the window was lost" if e % 2 == 0 else "the key just outside the window was seen"
        assert err <= 1.5e-2, f"request {e} of {L} tokens: {err:.3e} ({what}?)"
    from infero_b200.kernels import tc_gemm
    assert tc_gemm.error_flag() == 0


@pytest.mark.parametrize("H,Hkv,D", [(4, 2, 64), (7, 1, 128), (28, 4, 128)])
@pytest.mark.parametrize("window", [64, 200])
@pytest.mark.parametrize("P", [16, 64])
def test_window_edge_in_prefill_attention_on_tensor_memory(H, Hkv, D, window, P):
    """The same for prompt portions, at the rows where an off-by-one would hide: the first row after a
    cut, the last row of a block of 128 rows, the first row of the next block, the last row of the
    portion.  Requests come in pairs: key p - W + 1 dominant (must be seen) and key p - W dominant
    (must not).  Pages that lie wholly before the portion's window are not held (-1)."""
    from infero_b200.kernels import attention as A
    dt = torch.bfloat16
    portions = [(0, 300), (300, 260), (window + 13, 2), (511, 130)]
    if H >= 28:
        portions = [(0, 700), (300, 500), (window + 13, 2), (511, 130)]      # enough blocks for two heads per CTA
    lens = [pn for pn in portions for _ in (0, 1)]
    totals = [o + n for o, n in lens]
    table, kc, vc, Ks, Vs = _paged_requests(totals, Hkv, D, P, dt, 3, [o - window + 1 for o, _ in lens])
    T = sum(n for _, n in lens)
    scale = 1.0 / math.sqrt(D)
    qkv = _rand((T, (H + 2 * Hkv) * D), dt, 7)             # q sits in front of a wider row, as in the model
    q = qkv[:, :H * D]
    checked = []
    t0 = 0
    for e, (o, n) in enumerate(lens):
        for i in sorted({0, 127, 128, 255, 256, n - 1}):
            p = o + i
            j = p - window + 1 if e % 2 == 0 else p - window
            if i >= n or j < 0:
                continue
            kk = Ks[e][j, 0].float()
            qkv[t0 + i, :D] = (kk * (7.0 / scale / float(kk @ kk))).to(dt)
            checked.append((e, i, t0 + i))
        t0 += n
    assert len(checked) >= 20
    positions = torch.tensor([o + i for o, n in lens for i in range(n)], dtype=torch.int32, device=DEV)
    entry = torch.tensor([e for e, (_, n) in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    out = torch.zeros((T, H * D), dtype=dt, device=DEV)
    assert A.prefill_tc_supported(q, out, D, P)
    A.attention_any(q, out, kc, vc, table.to(DEV), entry, positions, H, Hkv, D, P, window, scale,
                    q_lens=[n for _, n in lens], pos0=[o for o, _ in lens])
    rows = {t for _, _, t in checked}
    t = 0
    for e, (o, n) in enumerate(lens):
        for i in range(n):
            if t in rows or i % 37 == 0:
                L = o + i + 1
                ref = _attention_ref(qkv[t, :H * D].double().cpu().view(H, D), Ks[e][:L].double().cpu(),
                                     Vs[e][:L].double().cpu(), scale, window)
                err = float((out[t].double().cpu().view(H, D) - ref).abs().max() / ref.abs().max())
                what = "" if t not in rows else (" (the oldest key inside the window was lost?)" if e % 2 == 0
                                                 else " (the key just outside the window was seen?)")
                assert err <= 1.5e-2, f"request {e} (cached {o}), row {i}: {err:.3e}{what}"
            t += 1
    from infero_b200.kernels import tc_gemm
    assert tc_gemm.error_flag() == 0


def test_consumers_add_up_partial_products():
    """The fused consumers of split-K partial sums against the plain sum."""
    from infero_b200 import kernels as Kn
    S, T, d, ff = 5, 6, 200, 300
    part = _rand((S, T, d), torch.float32, 1)
    bias = _rand((d,), torch.bfloat16, 2)
    w = _rand((d,), torch.bfloat16, 3) + 1
    x = _rand((T, d), torch.float32, 4)
    v = x.double() + part.double().sum(0) + bias.double()
    ref = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + 1e-5) * w.double()
    out = torch.empty((T, d), dtype=torch.bfloat16, device=DEV)
    Kn.add_rmsnorm(x, Kn.Partials(part, bias), w, 1e-5, out)
    assert float((x.double() - v).abs().max()) <= 1e-5
    assert float((out.double() - ref).abs().max() / ref.abs().max()) <= 5e-3
    gu = _rand((S, T, 2 * ff), torch.float32, 5)
    act = torch.empty((T, ff), dtype=torch.bfloat16, device=DEV)
    Kn.swiglu(Kn.Partials(gu), act)
    g, u = gu.double().sum(0)[:, 0::2], gu.double().sum(0)[:, 1::2]
    ref = g / (1 + torch.exp(-g)) * u
    assert float((act.double() - ref).abs().max() / ref.abs().max()) <= 5e-3
    # rotary + cache append from partial sums equals the two-step way
    H, Hkv, D, P, Tn = 6, 2, 48, 16, 5
    width = (H + 2 * Hkv) * D
    part = _rand((3, Tn, width), torch.float32, 6)
    bias = _rand((width,), torch.bfloat16, 7)
    positions = torch.tensor([3, 4, 40, 0, 17], dtype=torch.int32, device=DEV)
    entry = torch.tensor([0, 0, 1, 2, 1], dtype=torch.int32, device=DEV)
    table = torch.tensor([[2, -1, -1], [5, 1, 7], [3, -1, -1]], dtype=torch.int32, device=DEV)
    inv = torch.from_numpy((10000.0 ** (-2.0 * np.arange(D // 2) / D)).astype(np.float32)).to(DEV)
    kc1 = torch.zeros((8, Hkv, P, D), dtype=torch.float32, device=DEV); vc1 = torch.zeros_like(kc1)
    kc2 = torch.zeros_like(kc1); vc2 = torch.zeros_like(kc1)
    q1 = torch.empty((Tn, H * D), dtype=torch.float32, device=DEV)
    Kn.rope_cache_partials(Kn.Partials(part, bias), q1, positions, entry, table, inv, kc1, vc1, H, Hkv, D, P)
    qkv = (part.sum(0) + bias.float()).contiguous()
    Kn.rope_cache(qkv, positions, entry, table, inv, kc2, vc2, H, Hkv, D, P)
    assert float((q1 - qkv[:, :H * D]).abs().max()) <= 2e-5
    assert float((kc1 - kc2).abs().max()) <= 2e-5 and float((vc1 - vc2).abs().max()) <= 2e-5
    assert int((kc1 != 0).any(-1).sum()) == Tn * Hkv


# ---- sampling ------------------------------------------------------------------------------------
def test_argmax_lowest_index_wins_ties():
    from infero_b200 import kernels as Kn
    V = 152_064 + 3
    z = _rand((3, V), torch.float32, 1)
    z[0, 77] = z[0, 150_000] = 9.0
    z[1, V - 1] = 11.0
    z[2] = -float("inf")
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    Kn.argmax(z, out)
    assert out.tolist() == [77, V - 1, 0]


def _host_sample(z, temp, top_k, top_p, u):
    """crates/model/src/sampling.rs:169-235 restated on the host in 64-bit."""
    idx = np.argsort(-z, kind="stable")[:top_k]
    zz = z[idx].astype(np.float64)
    w = np.exp((zz - zz[0]) / max(temp, 1e-5))
    total = w.sum()
    p = min(max(top_p, 1e-4), 1.0)
    keep = len(w)
    acc = 0.0
    for i, wi in enumerate(w):
        acc += wi
        if acc >= p * total:
            keep = i + 1
            break
    w = w[:keep]
    r = u * w.sum()
    for i, wi in enumerate(w):
        r -= wi
        if r <= 0:
            return int(idx[i])
    return int(idx[keep - 1])


@pytest.mark.parametrize("V,ties", [(5003, False), (152064, False), (40001, True)])
def test_sample_matches_host_statement(V, ties):
    """Small vocabularies take one block per row; large ones go through blocks per chunk of 8,192
    logits first.  With ties: values from a handful of levels, so that the k-th largest is shared by
    many tokens in many chunks and the lowest tokens must win."""
    from infero_b200 import kernels as Kn
    R = 24
    rng = np.random.default_rng(5)
    zn = rng.normal(size=(R, V)).astype(np.float32) * 3
    if ties:
        zn = np.round(zn * 2) / 2
    z = torch.from_numpy(zn).to(DEV)
    temp = torch.tensor([0.7, 1.0, 0.3] * 8, dtype=torch.float32, device=DEV)
    top_k = torch.tensor([20, 50, 5, 1000] * 6, dtype=torch.int32, device=DEV)
    top_p = torch.tensor([0.8, 1.0, 0.5, 0.95, 0.9, 0.3] * 4, dtype=torch.float32, device=DEV)
    draw = torch.from_numpy(rng.random(R)).to(DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    Kn.sample(z, temp, top_k, top_p, draw, out)
    zh = z.cpu().numpy()
    for r in range(R):
        want = _host_sample(zh[r], float(temp[r]), int(top_k[r]), float(top_p[r]), float(draw[r]))
        assert int(out[r]) == want, f"row {r}"


def _host_penalty(logits: np.ndarray, history, penalty: float, window: int, greedy: bool) -> np.ndarray:
    """The reference's repetition penalty in NumPy, float32 like its logits
    (crates/model/src/sampling.rs:249-298): over the last ``window`` tokens of the history a positive
    logit is divided by the penalty and any other multiplied by it; the greedy scan marks tokens in a
    bitset (:256-271), so each distinct token is penalised once, while the sampling path walks the
    history (:284-297) and penalises once per occurrence."""
    out = logits.astype(np.float32).copy()
    pen = np.float32(penalty)
    if penalty == 1.0 or not len(history):
        return out
    recent = list(history[max(0, len(history) - window):])
    for t in (sorted(set(recent)) if greedy else recent):
        if t < out.size:
            out[t] = out[t] / pen if out[t] > 0 else out[t] * pen
    return out


def test_the_references_own_sampler_cases():
    """The inputs and expected picks of the reference's sampler tests
    (crates/model/src/sampling.rs:350-433), through the device sampler."""
    from infero_b200.sampling import SamplingParams, sample_rows
    from infero_b200.sampling.sampler import RowSampler

    def pick(logits, params, history=()):
        z = torch.tensor([logits], dtype=torch.float32, device=DEV)
        return sample_rows(z, [RowSampler(params)], [list(history)])[0]

    # greedy_takes_the_argmax (:350-355)
    assert pick([0.1, 5.0, -2.0, 4.9], SamplingParams.greedy()) == 1
    # top_k_1_is_greedy_even_at_temperature (:357-368)
    s = RowSampler(SamplingParams(temperature=2.0, top_k=1))
    for _ in range(20):
        z = torch.tensor([[0.1, 5.0, -2.0]], dtype=torch.float32, device=DEV)
        assert sample_rows(z, [s], [[]])[0] == 1
    # top_p_confines_sampling_to_the_nucleus (:388-405): one token holds nearly all the mass
    logits = [0.0] * 100
    logits[7] = 20.0
    s = RowSampler(SamplingParams(temperature=1.0, top_p=0.9, top_k=100, repetition_penalty=1.0, seed=1))
    for _ in range(50):
        z = torch.tensor([logits], dtype=torch.float32, device=DEV)
        assert sample_rows(z, [s], [[]])[0] == 7
    # repetition_penalty_demotes_recent_tokens (:407-419)
    p = SamplingParams(temperature=0.0, repetition_penalty=2.0, repetition_window=8)
    assert pick([1.0, 1.1, 1.0], p) == 1
    assert pick([1.0, 1.1, 1.0], p, [1]) != 1
    assert pick([1.0, 1.1, 1.0], p, [1]) == 0           # the tie goes to the lowest index (:302-310)
    # negative_logits_are_penalised_downward (:421-433)
    p = SamplingParams(temperature=0.0, repetition_penalty=2.0)
    assert pick([-1.0, -1.5], p) == 0
    assert pick([-1.0, -1.5], p, [0]) == 1
    # selection_picks_the_same_top_k_as_a_sort (:326-348): 200 draws stay inside the true top 20
    logits = [((i * 7919) % 5000) * 0.01 for i in range(5000)]
    allowed = set(np.argsort(-np.asarray(logits, dtype=np.float32), kind="stable")[:20].tolist())
    s = RowSampler(SamplingParams(temperature=1.0, top_k=20, top_p=1.0, repetition_penalty=1.0, seed=9))
    z = torch.tensor([logits], dtype=torch.float32, device=DEV)
    for _ in range(200):
        assert sample_rows(z.clone(), [s], [[]])[0] in allowed
    # a_seed_makes_sampling_reproducible (:370-386)
    logits = [i * 0.1 for i in range(64)]
    runs = []
    for _ in range(2):
        s = RowSampler(SamplingParams(seed=42, temperature=1.0, top_k=64, top_p=1.0, repetition_penalty=1.0))
        z = torch.tensor([logits], dtype=torch.float32, device=DEV)
        runs.append([sample_rows(z.clone(), [s], [[]])[0] for _ in range(32)])
    assert runs[0] == runs[1] and len(set(runs[0])) > 4


def test_penalty_from_the_device_history_equals_the_host_statement():
    """Rows whose generated tokens live in a ring on the device (appended by keep_tokens) against a
    NumPy statement of the reference's rule over the same histories: windows shorter and longer than the history, a
    ring that has wrapped, greedy rows (once per distinct token) beside sampled ones (once per
    occurrence), a row without a penalty."""
    from infero_b200 import kernels as Kn
    from infero_b200.sampling import SamplingParams
    from infero_b200.sampling.sampler import RowSampler
    V, W, slots_n = 777, 32, 6
    rng = np.random.default_rng(11)
    lens = [0, 5, 31, 32, 50, 200]                       # tokens generated so far, per slot
    hists = [[int(t) for t in rng.integers(0, 40, size=n)] for n in lens]      # few distinct tokens: many repeats
    ring = torch.zeros((slots_n, W), dtype=torch.int32, device=DEV)
    ring_len = torch.zeros(slots_n, dtype=torch.int32, device=DEV)
    # fill the rings the way the engine does: one keep_tokens per step
    for step in range(max(lens)):
        rows = [s for s in range(slots_n) if step < lens[s]]
        g = torch.tensor([hists[s][step] for s in rows], dtype=torch.int32, device=DEV)
        info = torch.tensor(rows + [0] * len(rows), dtype=torch.int32, device=DEV)
        Kn.keep_tokens(g, None, info, torch.empty(len(rows), dtype=torch.int32, device=DEV),
                       torch.zeros(slots_n, dtype=torch.int32, device=DEV), ring, ring_len)
    assert ring_len.tolist() == lens
    params = [SamplingParams(temperature=0.0, repetition_penalty=1.3, repetition_window=8),
              SamplingParams(temperature=0.7, repetition_penalty=1.1, repetition_window=16),
              SamplingParams(temperature=0.0, repetition_penalty=1.0),
              SamplingParams(temperature=0.9, repetition_penalty=1.25, repetition_window=32),
              SamplingParams(temperature=0.0, repetition_penalty=1.05, repetition_window=20),
              SamplingParams(temperature=0.5, repetition_penalty=1.2, repetition_window=32)]
    z0 = torch.from_numpy(rng.normal(size=(slots_n, V)).astype(np.float32) * 2).to(DEV)
    want = torch.from_numpy(np.stack([_host_penalty(z0[r].cpu().numpy(), hists[r], params[r].repetition_penalty,
                                                    params[r].repetition_window, params[r].is_greedy())
                                      for r in range(slots_n)])).to(DEV)
    # the other route of the product (pairs worked out on the host, applied by apply_penalty) gives the same
    via_pairs = z0.clone()
    pairs = [RowSampler(p).penalty_pairs(h) for p, h in zip(params, hists)]
    width = max(len(p) for p in pairs)
    toks = np.full((slots_n, width), -1, dtype=np.int32)
    cnts = np.zeros((slots_n, width), dtype=np.int32)
    for r, p in enumerate(pairs):
        for i, (t, c) in enumerate(p):
            toks[r, i], cnts[r, i] = t, c
    Kn.apply_penalty(via_pairs, torch.from_numpy(toks).to(DEV), torch.from_numpy(cnts).to(DEV),
                     torch.tensor([p.repetition_penalty for p in params], dtype=torch.float32, device=DEV))
    assert torch.equal(via_pairs, want)
    got = z0.clone()
    info = torch.tensor(list(range(slots_n)) + [0 if p.is_greedy() else 1 for p in params], dtype=torch.int32, device=DEV)
    Kn.apply_penalty_ring(got, info, torch.tensor([p.repetition_penalty for p in params], dtype=torch.float32, device=DEV),
                          torch.tensor([p.repetition_window for p in params], dtype=torch.int32, device=DEV), ring, ring_len)
    assert torch.equal(got, want)
    assert not torch.equal(got, z0)
