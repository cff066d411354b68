"""The W8A8 part of the oracle against the reference's own CPU kernels (its scales, quantise + packing and fused
dequantisation compiled from its sources), and the pure host functions of the typed W8A8 API."""
import ctypes as C

import numpy as np
import pytest

from conftest import bits
from oracle.harness import Reference, make_activations
from rknpu2_matmul_open_b200 import capi

needs_ref = pytest.mark.skipif(not Reference.available(), reason="reference checker not built")


def w8_weights(K, N, seed):
    rng = np.random.default_rng(seed)
    B = rng.integers(-127, 128, size=(K, N), dtype=np.int8)
    B[rng.random((K, N)) < 0.01] = -128
    return B, rng.uniform(1e-3, 2e-2, size=N).astype(np.float32)


def special_rows(A):
    """Rows that exercise the scale rules: all zero, one tiny value whose scale underflows, exact rounding ties."""
    M, K = A.shape
    if M >= 2:
        A[1, :] = 0
    if M >= 3:
        A[2, :] = 0
        A[2, K // 2] = 1e-45 if A.dtype == np.float32 else 1
    if M >= 4:
        A[3, :] = np.where(np.arange(K) % 2, 63.5, -0.5).astype(np.float32) if A.dtype == np.float32 else A[3, :]
        if A.dtype == np.float32:
            A[3, 0] = 127.0
    return A


@needs_ref
@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("shape", [(1, 33, 5), (5, 257, 70), (16, 2048, 96), (37, 1000, 131)], ids=lambda s: "x".join(map(str, s)))
def test_oracle_matches_the_reference_cpu_kernels(oracle, shape, dtype):
    ref = Reference()
    M, K, N = shape
    B, sw = w8_weights(K, N, seed=K)
    A = make_activations(M, K, seed=N, dtype=dtype)
    A = special_rows(A.view(np.uint16) if dtype == "f16" else A) if dtype == "f32" else A
    if dtype == "f16" and M >= 3:
        A[1, :] = 0
        A[2, :] = 0
        A[2, 7] = 0x0001                      # the smallest binary16 subnormal: its scale is far below FLT_MIN
    for static in (None, np.linspace(0.01, 0.3, M).astype(np.float32)):
        a = oracle.w8_linear(A, B, sw, static)
        b = ref.w8_linear(A, B, sw, static)
        assert a["rc"] == 0 and b["rc"] == 0
        assert np.array_equal(bits(a["scales"]), bits(b["scales"]))
        assert np.array_equal(a["codes"], b["codes"])
        assert np.array_equal(a["acc"], b["acc"])
        assert np.array_equal(bits(a["out"]), bits(b["out"]))


@needs_ref
def test_non_finite_activations_propagate_as_in_the_reference(oracle):
    ref = Reference()
    M, K, N = 4, 64, 8
    B, sw = w8_weights(K, N, seed=3)
    A = make_activations(M, K, seed=3, dtype="f32")
    A[0, 5] = np.nan            # ignored by the maximum, quantised to +127
    A[1, 9] = np.inf            # scale inf -> inverse 0: finite values give 0, the infinity NaN -> 127
    A[2, 3] = -np.inf
    a, b = oracle.w8_linear(A, B, sw), ref.w8_linear(A, B, sw)
    assert np.array_equal(bits(a["scales"]), bits(b["scales"]))
    assert np.array_equal(a["codes"], b["codes"])
    assert a["codes"][0, 5] == 127 and a["codes"][1, 9] == 127 and a["codes"][2, 3] == 127
    assert np.array_equal(a["acc"], b["acc"])
    fin = np.isfinite(a["out"])
    assert np.array_equal(fin, np.isfinite(b["out"])) and np.array_equal(bits(a["out"][fin]), bits(b["out"][fin]))


def test_int32_sums_wrap_modulo_2_32(oracle):
    # include/rk_npu_quant_matmul.h:335-340: sums are exact modulo 2^32
    K = 140000
    q = np.full((1, K), 127, np.int8)
    B = np.full((K, 2), 127, np.int8)
    B[:, 1] = -128
    acc = np.zeros((1, 2), np.int32)
    oracle.lib.orc_gemm_i32(q.ctypes.data_as(C.c_void_p), B.ctypes.data_as(C.c_void_p), 1, K, 2, acc.ctypes.data_as(C.c_void_p))
    exact = np.array([127 * 127 * K, -128 * 127 * K], np.int64)
    assert exact[0] > 2**31 and np.array_equal(acc[0], exact.astype(np.int32))


@needs_ref
def test_k_partition_query_matches_the_reference():
    lib = capi.load()
    ref = Reference()
    rng = np.random.default_rng(0)
    cases = [(1, 1, 1), (4, 9000, 3100), (5, 9000, 3100), (5, 8192, 4096), (5, 8192, 3073), (8, 6000, 2080), (8, 6000, 3072),
             (0, 5, 5), (3, 0, 1), (3, 5, 0), (3, 5, 6)]
    cases += [(int(rng.integers(1, 40)), int(k), int(rng.integers(1, k + 1))) for k in rng.integers(1, 12000, 300)]
    for M, K, kt in cases:
        assert lib.rk_npu_matmul_k_partition_query(M, K, kt) == ref.k_partition_query(M, K, kt), (M, K, kt)


def test_memory_queries_and_argument_errors():
    lib = capi.load()
    from rknpu2_matmul_open_b200 import w8a8
    out = capi.MatmulWeightRequirements()
    cfg = capi.MatmulWeightConfig(4096, 1000, 1024)
    assert lib.rk_npu_f16i8f16_weights_memory_query(C.byref(cfg), C.byref(out)) == 0
    assert out.scale_bytes == 4000 and out.wave_count == 4 and out.packed_b_bytes >= 4096 * 1000 and out.bytes == out.packed_b_bytes + 4000
    assert lib.rk_npu_i8i8i32_weights_memory_query(C.byref(cfg), C.byref(out)) == 0 and out.scale_bytes == 0
    for bad in (capi.MatmulWeightConfig(0, 8, 1), capi.MatmulWeightConfig(8, 0, 1), capi.MatmulWeightConfig(8, 8, 0), capi.MatmulWeightConfig(8, 8, 9)):
        assert lib.rk_npu_f32i8f32_weights_memory_query(C.byref(bad), C.byref(out)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_f32i8f32_weights_memory_query(None, C.byref(out)) == capi.RK_NPU_ERR_PARAM
    req = capi.MatmulWorkspaceRequirements()
    s = w8a8.default_strategy(w8a8.F16_DYNAMIC, 33, 1000, 4096, k_tile=1024)
    assert lib.rk_npu_matmul_workspace_memory_query(C.byref(s), C.byref(req)) == 0
    assert req.wave_count == 4 and req.bytes == req.input_bytes + req.output_bytes + req.control_bytes and req.output_bytes == 33 * 1000 * 2
    for field, value in (("M", 0), ("k_tile", 0), ("k_tile", 4097), ("n_tile", 3073), ("a_layout", 4), ("c_layout", 3), ("npu_core_mask", 5),
                         ("cpu_core_mask", 0), ("cpu_threads", 2), ("op_kind", 5)):
        t = w8a8.default_strategy(w8a8.F16_DYNAMIC, 33, 1000, 4096)
        setattr(t, field, value)
        assert lib.rk_npu_matmul_workspace_memory_query(C.byref(t), C.byref(req)) == capi.RK_NPU_ERR_PARAM, field
        assert lib.rk_npu_matmul_workspace_create(None, C.byref(t)) is None
    t = w8a8.default_strategy(w8a8.I8I8I32, 4, 64, 64)
    t.npu_core_mask, t.n_tile = 7, 64            # fewer column groups than device cores
    assert lib.rk_npu_matmul_workspace_memory_query(C.byref(t), C.byref(req)) == capi.RK_NPU_ERR_PARAM
