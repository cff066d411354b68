"""The exact int4 x int4 -> int32 operator (include/rk_npu_matmul_i4.h) through the C ABI: exact against the integer
formula of the reference's own board test (tests/test_i4.cpp: int64 dot products narrowed to int32), with the direct
call and with the producer callback, plus the argument and compatibility errors."""
import ctypes as C

import numpy as np
import pytest

from rknpu2_matmul_open_b200 import capi

pytestmark = pytest.mark.gpu


def make(lib, dom, M, N, K, k_tile=480, m_tile=128, rng=None):
    rng = rng or np.random.default_rng(K + N)
    B = rng.integers(-7, 8, size=(K, N), dtype=np.int8)
    A = rng.integers(-8, 8, size=(M, K), dtype=np.int8)
    w = lib.rk_npu_i4i4i32_weights_create(dom.handle, C.byref(capi.I4WeightConfig(K, N, k_tile)), B.ctypes.data)
    cfg = capi.I4Config()
    lib.rk_npu_i4_config_init(C.byref(cfg), M, N, K)
    cfg.k_tile, cfg.m_tile = k_tile, m_tile
    ws = lib.rk_npu_i4_workspace_create(dom.handle, C.byref(cfg))
    assert w and ws
    return A, B, w, ws, cfg


@pytest.mark.parametrize("shape", [(1, 1, 1), (7, 65, 513), (128, 1024, 4096), (300, 200, 1000), (16, 4096, 2048)], ids=lambda s: "x".join(map(str, s)))
def test_exact_sums_direct_and_through_the_producer(gpu, shape):
    lib = capi.load()
    _, dom, _ = gpu
    M, N, K = shape
    A, B, w, ws, cfg = make(lib, dom, M, N, K, k_tile=min(480, (K + 31) // 32 * 32), m_tile=min(128, M))
    exact = (A.astype(np.int64) @ B.astype(np.int64)).astype(np.int32)
    out = np.zeros((M, N), np.int32)
    t = capi.I4Timings()
    assert lib.rk_npu_i4i4i32_run(ws, w, A.ctypes.data, out.ctypes.data, C.byref(t)) == 0
    assert np.array_equal(out, exact) and t.total_us > 0 and t.submit_us > 0

    calls = []

    def producer(user, tile_ptr):
        tile = tile_ptr.contents
        calls.append((tile.k0, tile.m0, tile.rows, tile.k, tile.padded_k))
        # the tile arrives zeroed
        raw = np.ctypeslib.as_array(tile.dst, shape=(tile.bytes,))
        assert not raw.any()
        return lib.rk_npu_i4_pack_a_tile(tile_ptr, A.ctypes.data, K)

    out[:] = -1
    assert lib.rk_npu_i4i4i32_run_with_producer(ws, w, capi.I4_PRODUCER(producer), None, out.ctypes.data, None) == 0
    assert np.array_equal(out, exact)
    # K waves in increasing order, M panels in increasing order inside each
    expected = [(k0, m0, min(cfg.m_tile, M - m0), min(cfg.k_tile, K - k0), (min(cfg.k_tile, K - k0) + 31) // 32 * 32)
                for k0 in range(0, K, cfg.k_tile) for m0 in range(0, M, cfg.m_tile)]
    assert calls == expected
    # a producer that fails ends the run with its code
    assert lib.rk_npu_i4i4i32_run_with_producer(ws, w, capi.I4_PRODUCER(lambda u, t: capi.RK_NPU_ERR_IO), None, out.ctypes.data, None) == capi.RK_NPU_ERR_IO
    out[:] = 0
    assert lib.rk_npu_i4i4i32_run(ws, w, A.ctypes.data, out.ctypes.data, None) == 0 and np.array_equal(out, exact)   # still usable
    lib.rk_npu_i4_workspace_free(ws)
    lib.rk_npu_i4i4i32_weights_free(w)


def test_argument_and_compatibility_errors(gpu):
    lib = capi.load()
    ctx, dom, _ = gpu
    M, N, K = 9, 130, 700
    A, B, w, ws, cfg = make(lib, dom, M, N, K)
    out = np.zeros((M, N), np.int32)
    bad = A.copy()
    bad[4, 5] = 8
    assert lib.rk_npu_i4i4i32_run(ws, w, bad.ctypes.data, out.ctypes.data, None) == capi.RK_NPU_ERR_PARAM     # not masked
    bad[4, 5] = -9
    assert lib.rk_npu_i4i4i32_run(ws, w, bad.ctypes.data, out.ctypes.data, None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_i4i4i32_run(ws, None, A.ctypes.data, out.ctypes.data, None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_i4i4i32_run(ws, w, A.ctypes.data, None, None) == capi.RK_NPU_ERR_PARAM
    # weights of another K partition, weights of another domain
    other = lib.rk_npu_i4i4i32_weights_create(dom.handle, C.byref(capi.I4WeightConfig(K, N, 448)), B.ctypes.data)
    assert other and lib.rk_npu_i4i4i32_run(ws, other, A.ctypes.data, out.ctypes.data, None) == capi.RK_NPU_ERR_PARAM
    lib.rk_npu_i4i4i32_weights_free(other)
    dom2 = ctx.domain(5)
    foreign = lib.rk_npu_i4i4i32_weights_create(dom2.handle, C.byref(capi.I4WeightConfig(K, N, 480)), B.ctypes.data)
    assert foreign and lib.rk_npu_i4i4i32_run(ws, foreign, A.ctypes.data, out.ctypes.data, None) == capi.RK_NPU_ERR_DOMAIN
    lib.rk_npu_i4i4i32_weights_free(foreign)
    dom2.free()
    # creation: a code outside [-8,7], a bad key, an uncertified tile above 480 (all +7: 7 x 7 x 2048 saturates INT16)
    Bbad = B.copy()
    Bbad[0, 0] = 8
    assert not lib.rk_npu_i4i4i32_weights_create(dom.handle, C.byref(capi.I4WeightConfig(K, N, 480)), Bbad.ctypes.data)
    assert not lib.rk_npu_i4i4i32_weights_create(dom.handle, C.byref(capi.I4WeightConfig(K, N, 481)), B.ctypes.data)
    big = np.full((2048, 64), 7, np.int8)
    assert not lib.rk_npu_i4i4i32_weights_create(dom.handle, C.byref(capi.I4WeightConfig(2048, 64, 2048)), big.ctypes.data)
    small = np.zeros((2048, 64), np.int8)
    ok = lib.rk_npu_i4i4i32_weights_create(dom.handle, C.byref(capi.I4WeightConfig(2048, 64, 2048)), small.ctypes.data)
    assert ok
    lib.rk_npu_i4i4i32_weights_free(ok)
    c2 = capi.I4Config()
    lib.rk_npu_i4_config_init(C.byref(c2), M, N, K)
    c2.m_tile = 129
    assert not lib.rk_npu_i4_workspace_create(dom.handle, C.byref(c2))
    lib.rk_npu_i4_workspace_free(ws)
    lib.rk_npu_i4i4i32_weights_free(w)
