"""Residual add + RMSNorm without a GPU: the oracle's restatement of the original's board-test expression
(tests/test_add_rmsnorm_f16.cpp:96-113) against an independent numpy evaluation, the block-8 layout helpers, and the
host-only entry points (configuration, size query, buffer views, argument errors)."""
import ctypes as C

import numpy as np
import pytest

from rknpu2_matmul_open_b200 import capi, rmsnorm


def board_inputs(M, D, seed):
    """The board test's distributions: x ~ N(0, 0.8) clamped to +-3, residual ~ N(0, 0.35) clamped to +-1.5,
    gamma a ramp from 0.75 to 1.25, all rounded to fp16."""
    rng = np.random.default_rng(seed)
    x = np.clip(rng.normal(0, 0.8, (M, D)), -3, 3).astype(np.float16)
    r = np.clip(rng.normal(0, 0.35, (M, D)), -1.5, 1.5).astype(np.float16)
    g = (0.75 + 0.5 * np.arange(D) / max(D - 1, 1)).astype(np.float16)
    return x.view(np.uint16), r.view(np.uint16), g.view(np.uint16)


def numpy_statement(x, r, g, eps):
    xs, rs, gs = x.view(np.float16), r.view(np.float16), g.view(np.float16)
    sums = (xs.astype(np.float32) + rs.astype(np.float32)).astype(np.float16)
    v = sums.astype(np.float64)
    variance = np.zeros(v.shape[0])
    for d in range(v.shape[1]):                 # in order of d, as the board test adds them
        variance += v[:, d] * v[:, d]
    with np.errstate(all="ignore"):
        inv = 1.0 / np.sqrt(variance / v.shape[1] + np.float64(np.float32(eps)))
        norm = (v * inv[:, None] * gs.astype(np.float64)).astype(np.float32).astype(np.float16)
    return sums.view(np.uint16), norm.view(np.uint16)


@pytest.mark.parametrize("M,D,eps", [(1, 4096, 1e-5), (128, 4096, 1e-5), (7, 64, 1e-6), (3, 8, 0.0), (2, 32768, 1e-3)])
def test_oracle_equals_the_numpy_statement(oracle, M, D, eps):
    x, r, g = board_inputs(M, D, 100 + M)
    if M > 1:
        x[1], r[1] = 0, 0                       # a zero row: inv = 1 / sqrt(eps) times 0 (eps = 0: NaN from 0 * inf)
    sums, norm = oracle.add_rmsnorm_f16(x, r, g, eps)
    want_sums, want_norm = numpy_statement(x, r, g, eps)
    assert np.array_equal(sums, want_sums)
    assert np.array_equal(norm, want_norm)
    # and the board test's own bars around it hold trivially
    err = np.abs(norm.view(np.float16).astype(np.float64) - want_norm.view(np.float16).astype(np.float64))
    assert np.nan_to_num(err).max() <= 0.04


def test_block8_layout_helpers():
    M, D = 5, 48
    rows = np.arange(M * D, dtype=np.uint16).reshape(M, D)
    flat = rmsnorm.to_block8(rows)
    for m, d in [(0, 0), (4, 47), (2, 9), (3, 16)]:
        assert flat[((d // 8) * M + m) * 8 + d % 8] == rows[m, d]      # tests/test_add_rmsnorm_f16.cpp:26-28
    assert np.array_equal(rmsnorm.from_block8(flat, M, D), rows)


def test_host_entry_points(lib):
    c = rmsnorm.default_config(128, 4096)
    assert (c.M, c.D, c.timeout_ms) == (128, 4096, 6000) and c.eps == np.float32(1e-5)
    sizes = rmsnorm.query(c)
    assert (sizes.tensor_bytes, sizes.weight_bytes, sizes.num_tasks) == (128 * 4096 * 2, 4096 * 2, 1)
    assert (sizes.internal_bytes, sizes.regcmd_bytes, sizes.task_bytes) == (0, 0, 0)
    for M, D, eps in [(0, 4096, 1e-5), (65537, 4096, 1e-5), (1, 4, 1e-5), (1, 4100, 1e-5), (1, 32776, 1e-5), (1, 4096, -1.0),
                      (1, 4096, float("nan")), (1, 4096, float("inf"))]:
        bad = rmsnorm.default_config(M, D)
        bad.eps = eps
        out = capi.AddRmsNormSizes()
        assert lib.rk_npu_add_rmsnorm_f16_query(C.byref(bad), C.byref(out)) == capi.RK_NPU_ERR_PARAM, (M, D, eps)
    assert lib.rk_npu_add_rmsnorm_f16_query(None, C.byref(capi.AddRmsNormSizes())) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_add_rmsnorm_f16_query(C.byref(c), None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_add_rmsnorm_f16_plan_create(None, C.byref(c), None) is None
    lib.rk_npu_add_rmsnorm_f16_plan_free(None)
    assert lib.rk_npu_add_rmsnorm_f16_run(None, None, None, None, None, None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_b200_add_rmsnorm_f16_enqueue(None, 1, 0, None, None, None, None, None) == capi.RK_NPU_ERR_PARAM


def test_buffer_views_and_argument_errors(lib):
    # views are arithmetic on the struct (src/rk_npu_core.cpp:318-331): no device needed
    host = (C.c_uint8 * 4096)()
    base = capi.Mem(handle=7, flags=(1 << 0) | (1 << 3) | (1 << 4), obj_addr=0x10000, dma_addr=0x10000,
                    vaddr=C.addressof(host), size=4096, offset=0, capacity=4096, ctx_id=99, iommu_domain_id=3)
    view, inner = capi.Mem(), capi.Mem()
    assert lib.rk_npu_mem_view(C.byref(base), 1024, 2048, C.byref(view)) == capi.RK_NPU_OK
    assert (view.dma_addr, view.vaddr, view.size, view.offset, view.capacity) == (0x10400, C.addressof(host) + 1024, 2048, 1024, 4096)
    assert view.flags == (1 << 2) | (1 << 3) | (1 << 4)            # VIEW | MAPPED | CACHEABLE, not OWN
    assert (view.handle, view.ctx_id, view.iommu_domain_id) == (7, 99, 3)
    assert lib.rk_npu_mem_view(C.byref(view), 2047, 1, C.byref(inner)) == capi.RK_NPU_OK and inner.offset == 3071
    for offset, size in [(0, 0), (4097, 1), (1, 4096), (4096, 1)]:
        assert lib.rk_npu_mem_view(C.byref(base), offset, size, C.byref(inner)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_view(None, 0, 1, C.byref(inner)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_view(C.byref(base), 0, 1, None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_alloc(None, 64, 0, C.byref(inner)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_free(None, C.byref(inner)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_sync(None, C.byref(base), 1) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_import_dmabuf(None, 0, None, 64, 0, C.byref(inner)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_export_dmabuf(None, C.byref(base), None) == capi.RK_NPU_ERR_PARAM
