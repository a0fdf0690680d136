"""How the native code cuts work into blocks (pure host functions of the kernel library; no GPU):
the few-token products' splits of K, the cluster-summed variant's limits, decode attention's splits."""
from ctypes import byref, c_int, c_longlong

import pytest

from infero_b200 import kernels as K


def _plan(M, N, Kd, sms=148):
    s, per, ws = c_int(0), c_int(0), c_longlong(0)
    K.lib().infero_gemm_tc_plan(c_int(M), c_int(N), c_int(Kd), c_int(sms), byref(s), byref(per), byref(ws))
    return s.value, per.value, ws.value


def _plan_cluster(M, N, Kd, sms=148):
    s, per = c_int(0), c_int(0)
    K.lib().infero_gemm_tc_plan_cluster(c_int(M), c_int(N), c_int(Kd), c_int(sms), byref(s), byref(per))
    return s.value, per.value


SHAPES = [(8, 3584, 3584), (8, 3584, 18944), (1, 5120, 5120), (64, 5120, 13824), (8, 896, 4864), (8, 896, 896),
          (3, 128, 320), (16, 256, 616), (200, 1000, 2048), (8, 37888, 3584), (8, 152064, 3584)]


@pytest.mark.parametrize("M,N,Kd", SHAPES)
def test_the_splits_cover_k_and_the_workspace_holds_them(M, N, Kd):
    s, per, ws = _plan(M, N, Kd)
    total_kt = -(-Kd // 64)
    assert 1 <= s <= 16 and per >= 1
    assert (s - 1) * per < total_kt <= s * per, "every split has k-tiles and together they cover K"
    assert ws == (s * M * N * 4 if s > 1 else 0)


@pytest.mark.parametrize("M,N,Kd", SHAPES)
def test_a_grid_of_clusters_leaves_room(M, N, Kd):
    """At most 8 splits (one cluster), never more than the free plan, and about a fifth of the block slots
    left free unless a single split per tile already takes more."""
    s, per = _plan_cluster(M, N, Kd)
    free_s, _, _ = _plan(M, N, Kd)
    total_kt = -(-Kd // 64)
    tiles = -(-N // 128)
    assert 1 <= s <= min(8, free_s)
    assert (s - 1) * per < total_kt <= s * per
    assert s == 1 or tiles * s <= int(0.82 * 296)


def test_the_measured_shapes_get_the_measured_plans():
    assert _plan_cluster(8, 3584, 3584)[0] == 8 and _plan_cluster(8, 3584, 18944)[0] == 8      # hidden 3584: 28 tiles x 8
    assert _plan_cluster(8, 5120, 5120)[0] == 6 and _plan_cluster(8, 5120, 13824)[0] == 6      # hidden 5120: 40 tiles x 6
    assert _plan(8, 37888, 3584)[0] == 1                                                       # gate/up: a tile per block


@pytest.mark.parametrize("n_tok,n_kv,group,visible", [(1, 4, 7, 4096), (8, 4, 7, 4096), (64, 4, 7, 4096), (8, 8, 5, 131072),
                                                     (3, 1, 20, 17), (256, 2, 2, 700), (1, 2, 7, 300)])
def test_decode_attention_splits_cover_the_keys(n_tok, n_kv, group, visible):
    chunk, splits = c_int(0), c_int(0)
    K.lib().infero_attn_plan_decode(c_int(n_tok), c_int(n_kv), c_int(group), c_int(visible), c_int(148), byref(chunk),
                                    byref(splits))
    assert chunk.value % 16 == 0 and chunk.value >= 256 or splits.value == 256
    assert 1 <= splits.value <= 256
    assert chunk.value * splits.value >= visible, "the splits cover every visible key"
    assert chunk.value * (splits.value - 1) < max(visible, 16), "and none of them is empty by plan"
