"""The typed W8A8 operators (int8 weights) through the C ABI against the oracle, bit for bit.

Covered: the five operator kinds, dynamic and static per-token scales, token counts below one tile, at tile edges
and over several tiles, K and N tails, zero rows and rows whose scale underflows, full-range int8 weights including
-128, sums that wrap modulo 2^32, one weight object shared by workspaces of different M, and the error behaviour of
include/rk_npu_quant_matmul.h (operator mismatch, incompatible key, foreign domain, bad static scales)."""
import ctypes as C

import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from oracle.harness import make_activations
from rknpu2_matmul_open_b200 import capi, w8a8

pytestmark = pytest.mark.gpu


def w8_weights(K, N, seed):
    rng = np.random.default_rng(seed)
    B = rng.integers(-127, 128, size=(K, N), dtype=np.int8)
    B[rng.random((K, N)) < 0.01] = -128
    return B, rng.uniform(1e-3, 2e-2, size=N).astype(np.float32)


def activations(M, K, seed, dtype):
    A = make_activations(M, K, seed=seed, dtype=dtype)
    if M >= 3:
        A[1, :] = 0
        A[2, :] = 0
        A[2, K // 2] = 0x0001 if dtype == "f16" else 1e-45     # the scale underflows (f32) or is subnormal (f16)
    return A


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("shape", [(1, 33, 5), (8, 4096, 4096), (16, 257, 70), (17, 1000, 131), (128, 2048, 384), (256, 640, 129),
                                   (300, 1057, 513), (1024, 512, 256), (520, 768, 9985)], ids=lambda s: "x".join(map(str, s)))
def test_dynamic_and_static(gpu, oracle, shape, dtype):
    _, dom, _ = gpu
    M, K, N = shape
    B, sw = w8_weights(K, N, seed=K + N)
    A = activations(M, K, seed=M, dtype=dtype)
    fam = "f16i8f16" if dtype == "f16" else "f32i8f32"
    w = w8a8.MatmulWeights(dom, fam, B, sw, k_tile=min(K, 1024))
    out_t = np.uint16 if dtype == "f16" else np.float32
    dyn = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.F16_DYNAMIC if dtype == "f16" else w8a8.F32_DYNAMIC, M, N, K, min(K, 1024)))
    sta = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.F16_STATIC if dtype == "f16" else w8a8.F32_STATIC, M, N, K, min(K, 1024)))
    out = np.full((M, N), 7, out_t)
    assert dyn.run_dynamic(w, A, out) == 0
    assert dyn.launch_count() == 2
    ref = oracle.w8_linear(A, B, sw)
    assert np.array_equal(bits(out), bits(ref["out"]))
    a_scale = np.linspace(0.01, 0.3, M).astype(np.float32)
    out[:] = 7
    assert sta.run_static(w, A, a_scale, out) == 0
    assert np.array_equal(bits(out), bits(oracle.w8_linear(A, B, sw, a_scale)["out"]))
    # the operator a workspace was made for is the only one it runs
    assert dyn.run_static(w, A, a_scale, out) == capi.RK_NPU_ERR_PARAM
    assert sta.run_dynamic(w, A, out) == capi.RK_NPU_ERR_PARAM
    bad = a_scale.copy()
    bad[M // 2] = 0
    assert sta.run_static(w, A, bad, out) == capi.RK_NPU_ERR_PARAM
    bad[M // 2] = np.inf
    assert sta.run_static(w, A, bad, out) == capi.RK_NPU_ERR_PARAM
    # second call on the same objects
    out[:] = 0
    assert dyn.run_dynamic(w, A, out) == 0 and np.array_equal(bits(out), bits(ref["out"]))
    for x in (dyn, sta, w):
        x.free()


@pytest.mark.parametrize("shape", [(1, 1, 1), (5, 100, 37), (64, 4096, 300), (260, 777, 129)], ids=lambda s: "x".join(map(str, s)))
def test_int8_activations_exact_sums(gpu, oracle, shape):
    _, dom, _ = gpu
    M, K, N = shape
    rng = np.random.default_rng(K)
    B, _ = w8_weights(K, N, seed=1)
    A = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    w = w8a8.MatmulWeights(dom, "i8i8i32", B)
    ws = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.I8I8I32, M, N, K))
    out = np.zeros((M, N), np.int32)
    assert ws.run_i8(w, A, out) == 0
    assert np.array_equal(out, (A.astype(np.int64) @ B.astype(np.int64)).astype(np.int32))
    ws.free()
    w.free()


def test_compressed_storage_constructors_give_the_plain_results(gpu, oracle):
    # include/rk_npu_quant_matmul.h:321-330: lossless storage of the same B, same run and free functions, same results
    _, dom, _ = gpu
    M, K, N = 20, 640, 200
    B, sw = w8_weights(K, N, seed=3)
    for dtype, fam, kind in (("f16", "f16i8f16", w8a8.F16_DYNAMIC), ("f32", "f32i8f32", w8a8.F32_DYNAMIC)):
        A = activations(M, K, seed=4, dtype=dtype)
        w = w8a8.MatmulWeights(dom, fam, B, sw, compress=True)
        ws = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(kind, M, N, K))
        out = np.zeros((M, N), np.uint16 if dtype == "f16" else np.float32)
        assert ws.run_dynamic(w, A, out) == 0
        assert np.array_equal(bits(out), bits(oracle.w8_linear(A, B, sw)["out"]))
        if fam == "f32i8f32":
            assert capi.load().rk_npu_f32i8f32_weights_compressed_layout_generation(w.handle) == 0      # stored uncompressed here
        ws.free(); w.free()
    rng = np.random.default_rng(6)
    A8 = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    w = w8a8.MatmulWeights(dom, "i8i8i32", B, compress=True)
    ws = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.I8I8I32, M, N, K))
    acc = np.zeros((M, N), np.int32)
    assert ws.run_i8(w, A8, acc) == 0
    assert np.array_equal(acc, A8.astype(np.int32) @ B.astype(np.int32))
    ws.free(); w.free()
    with pytest.raises(rk.W4A8Error):
        w8a8.MatmulWeights(dom, "f16i8f16", B, np.zeros(N, np.float32), compress=True)       # the same validation


def test_panel_recipes_run_like_any_other_and_invalid_ones_are_refused(gpu, oracle):
    # src/rk_npu_quant_matmul.cpp:167-177: a strategy that names panel layouts is valid where the original's device
    # plan takes it; the layouts describe that device's buffers, the results are the same
    _, dom, _ = gpu
    M, K, N = 48, 512, 200
    B, sw = w8_weights(K, N, seed=9)
    A = activations(M, K, seed=9, dtype="f16")
    w = w8a8.MatmulWeights(dom, "f16i8f16", B, sw)
    want = oracle.w8_linear(A, B, sw)["out"]
    for a_layout, c_layout in ((2, 0), (3, 0), (2, 1), (3, 2), (0, 1)):
        st = w8a8.default_strategy(w8a8.F16_DYNAMIC, M, N, K)
        st.a_layout, st.c_layout = a_layout, c_layout
        ws = w8a8.MatmulWorkspace(dom, st)
        out = np.zeros((M, N), np.uint16)
        assert ws.run_dynamic(w, A, out) == 0 and np.array_equal(out, want)
        ws.free()
    for rows, a_layout, c_layout in ((48, 2, 2), (48, 1, 1), (48, 0, 2), (44, 3, 0), (44, 2, 1)):
        st = w8a8.default_strategy(w8a8.F16_DYNAMIC, rows, N, K)
        st.a_layout, st.c_layout = a_layout, c_layout
        with pytest.raises(rk.W4A8Error):
            w8a8.MatmulWorkspace(dom, st)
    w.free()


def test_sums_wrap_modulo_2_32(gpu):
    # include/rk_npu_quant_matmul.h:335-340.  (-128) x (-128) x 131072 = 2^31 wraps to INT32_MIN.
    _, dom, _ = gpu
    M, K, N = 2, 131072, 40
    A = np.full((M, K), -128, np.int8)
    A[1, :] = 127
    B = np.full((K, N), -128, np.int8)
    B[:, 1] = 127
    w = w8a8.MatmulWeights(dom, "i8i8i32", B)
    ws = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.I8I8I32, M, N, K))
    out = np.zeros((M, N), np.int32)
    assert ws.run_i8(w, A, out) == 0
    exact = A.astype(np.int64) @ B.astype(np.int64)
    assert exact[0, 0] == 2**31 and out[0, 0] == -2**31
    assert np.array_equal(out, exact.astype(np.int32))
    ws.free()
    w.free()


def test_one_weight_object_many_workspaces_and_the_compatibility_rules(gpu, oracle):
    ctx, dom, _ = gpu
    K, N = 1536, 200
    B, sw = w8_weights(K, N, seed=5)
    w = w8a8.MatmulWeights(dom, "f32i8f32", B, sw, k_tile=512)
    for M in (1, 9, 40, 257):
        A = activations(M, K, seed=M, dtype="f32")
        ws = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.F32_DYNAMIC, M, N, K, 512))
        out = np.zeros((M, N), np.float32)
        assert ws.run_dynamic(w, A, out) == 0
        assert np.array_equal(bits(out), bits(oracle.w8_linear(A, B, sw)["out"]))
        ws.free()
    M = 4
    A = activations(M, K, seed=1, dtype="f32")
    out = np.zeros((M, N), np.float32)
    other_key = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.F32_DYNAMIC, M, N, K, 768))     # same shape, other K partition
    assert other_key.run_dynamic(w, A, out) == capi.RK_NPU_ERR_PARAM
    other_key.free()
    other_dom = ctx.domain(3)
    foreign = w8a8.MatmulWorkspace(other_dom, w8a8.default_strategy(w8a8.F32_DYNAMIC, M, N, K, 512))
    assert foreign.run_dynamic(w, A, out) == capi.RK_NPU_ERR_DOMAIN
    foreign.free()
    other_dom.free()
    w.free()
    # creation: bad scales, bad key
    assert not capi.load().rk_npu_f32i8f32_weights_create(dom.handle, C.byref(capi.MatmulWeightConfig(K, N, 512)), B.ctypes.data_as(C.c_void_p),
                                                          np.zeros(N, np.float32).ctypes.data_as(C.c_void_p))
    assert not capi.load().rk_npu_i8i8i32_weights_create(dom.handle, C.byref(capi.MatmulWeightConfig(K, N, K + 1)), B.ctypes.data_as(C.c_void_p))


def test_memory_accounting_returns_to_the_baseline(gpu):
    _, dom, _ = gpu
    before = dom.memory_stats()
    B, sw = w8_weights(512, 96, seed=2)
    w = w8a8.MatmulWeights(dom, "f16i8f16", B, sw)
    ws = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.F16_DYNAMIC, 12, 96, 512))
    mid = dom.memory_stats()
    assert mid.live_bytes > before.live_bytes
    ws.free()
    w.free()
    after = dom.memory_stats()
    assert after.live_bytes == before.live_bytes and after.creates - after.destroys == before.creates - before.destroys
