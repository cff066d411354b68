"""The routed-experts part of the oracle: its fused middle stage against the reference's own compiled routine
(src/rk_npu_moe_cpu.cpp, x86 form), nearest-even quantisation against its known answers, the whole operator against an
independent numpy restatement of the board test's reference (tests/test_moe_w8.cpp:27-46), and the host-only
entry points of the C ABI."""
import ctypes as C

import numpy as np
import pytest

from oracle.harness import Reference
from rknpu2_matmul_open_b200 import capi

needs_ref = pytest.mark.skipif(not Reference.available(), reason="reference checker not built")


def make_experts(H, I, E, seed):
    rng = np.random.default_rng(seed)
    return dict(gate_up=rng.integers(-127, 128, size=(E, H, 2 * I), dtype=np.int8),
                gate_up_scales=rng.uniform(2e-4, 6e-4, size=(E, 2 * I)).astype(np.float32),
                down=rng.integers(-127, 128, size=(E, I, H), dtype=np.int8),
                down_scales=rng.uniform(1e-3, 3e-3, size=(E, H)).astype(np.float32))


@needs_ref
@pytest.mark.parametrize("channels", [32, 64, 512])
def test_middle_row_equals_the_reference_routine(oracle, reference, channels):
    # sums and scales built like tests/test_moe_cpu.cpp:24-43 (W8 form), plus random rows and an all-zero row
    rng = np.random.default_rng(channels)
    n = np.arange(2 * channels)
    scales = (0.002 + (n % 11) * 0.00017).astype(np.float32)
    for row in range(33):
        hi = (n * 13 + row * 17) % 601 - 300
        lo = (n * 11 + row * 7) % 1001 - 500
        acc = (hi * 13 + lo).astype(np.int32) if row % 3 else rng.integers(-400000, 400000, size=2 * channels).astype(np.int32)
        sa = np.float32(0.015 + row * 0.0001)
        s_o, q_o = oracle.moe_middle_row(acc, sa, scales, mode=0)
        s_r, q_r = reference.moe_middle_row(acc, sa, scales)
        assert np.float32(s_o).tobytes() == np.float32(s_r).tobytes()
        assert np.array_equal(q_o, q_r)
        assert np.abs(q_o).max() == 127          # the row maximum maps to +-127
    zero = np.zeros(2 * channels, np.int32)
    for mode in (0, 1):
        s, q = oracle.moe_middle_row(zero, 0.1, scales, mode=mode)
        assert s == 1.0 and not q.any()          # src/rk_npu_moe_cpu.cpp:79-80: scale 1 for an all-zero row
    assert reference.moe_middle_row(zero, 0.1, scales)[0] == 1.0


def test_polynomial_and_exp_middle_rows_agree_to_rounding(oracle):
    rng = np.random.default_rng(5)
    acc = rng.integers(-300000, 300000, size=1024).astype(np.int32)
    ws = rng.uniform(2e-3, 4e-3, size=1024).astype(np.float32)
    s0, q0 = oracle.moe_middle_row(acc, 0.015, ws, mode=0)
    s1, q1 = oracle.moe_middle_row(acc, 0.015, ws, mode=1)
    assert abs(s0 - s1) <= 1e-6 * s0 and np.abs(q0.astype(int) - q1.astype(int)).max() <= 1


def test_nearest_even_row_quantisation(oracle):
    # the anchors of tests/test_moe_w8.cpp:107: ties go to the even code, unlike the dense path
    x = np.zeros((4, 64), np.float32)
    x[0, :8] = [127, -127, .5, 1.5, 2.5, -.5, -1.5, -2.5]
    x[1, :3] = [1e-3, -2e-3, 5e-4]
    x[3, 5] = 1e-45
    rc, q, s = oracle.moe_quantize_rows(x[:3])
    assert rc == 0
    assert q[0, :8].tolist() == [127, -127, 0, 2, 2, 0, -2, -2] and s[0] == 1.0
    assert q[1, 1] == -127 and s[1] == np.float32(2e-3) / np.float32(127)
    assert s[2] == 1.0 and not q[2].any()                      # zero row: scale 1
    assert oracle.moe_quantize_rows(x[3:4])[0] == 1            # the scale underflows to 0: rejected (src/rk_npu_moe_w8.cpp:324)
    x[1, 7] = np.nan
    assert oracle.moe_quantize_rows(x[:2])[0] == 1             # a non-finite element rejects the row
    # against numpy's rint (ties to even) on random rows
    rng = np.random.default_rng(1)
    y = rng.standard_normal((16, 96)).astype(np.float32) * 3
    rc, q, s = oracle.moe_quantize_rows(y)
    want_s = np.abs(y).max(axis=1) / np.float32(127)
    want_q = np.rint(np.clip(y * (np.float32(1) / want_s)[:, None], -127, 127)).astype(np.int8)
    assert rc == 0 and np.array_equal(s, want_s) and np.array_equal(q, want_q)


def numpy_moe(ex, shared, top, codes, scales, ids, routes):
    """tests/test_moe_w8.cpp:27-46 in numpy (sigmoid through exp, float64-free: every step in fp32)."""
    E, H, I2 = ex["gate_up"].shape
    I = I2 // 2
    rows = codes.shape[0]
    out = np.zeros((rows, H), np.float32)
    for r in range(rows):
        for slot in range(top + shared):
            e = int(ids[r, slot]) if slot < top else E - 1
            c = np.float32(routes[r, slot]) if slot < top else np.float32(1)
            acc = codes[r].astype(np.int64) @ ex["gate_up"][e].astype(np.int64)
            g = (acc.astype(np.float32) * np.float32(scales[r])) * ex["gate_up_scales"][e]
            hidden = (g[:I] / (np.float32(1) + np.exp(-g[:I]))) * g[I:]
            m = np.abs(hidden).max()
            s = m / np.float32(127) if m else np.float32(1)
            q = np.rint(np.clip(hidden * (np.float32(1) / s), -127, 127)).astype(np.int64)
            value = ((q @ ex["down"][e].astype(np.int64)).astype(np.float32) * s) * ex["down_scales"][e]
            out[r] = (value.astype(np.float64) * np.float64(c) + out[r].astype(np.float64)).astype(np.float32)   # one rounding: fma
    return out


@pytest.mark.parametrize("shape", [(64, 32, 3, 1, 2, 5), (96, 64, 5, 0, 3, 9)], ids=lambda s: "x".join(map(str, s)))
def test_whole_operator_against_numpy(oracle, shape):
    H, I, routed, shared, top, rows = shape
    ex = make_experts(H, I, routed + shared, seed=7)
    rng = np.random.default_rng(8)
    codes = rng.integers(-127, 128, size=(rows, H), dtype=np.int8)
    scales = rng.uniform(0.01, 0.05, size=rows).astype(np.float32)
    ids = rng.integers(0, routed, size=(rows, top)).astype(np.int32)
    routes = rng.uniform(0.1, 0.9, size=(rows, top)).astype(np.float32)
    ids[0, :] = 0                      # duplicates are summed in slot order
    routes[1, 0] = 0                   # a zero coefficient leaves the route out
    want = numpy_moe(ex, shared, top, codes, scales, ids, routes)
    rc, got = oracle.moe_run(ex, shared, top, codes, scales, ids, routes, mode=0)
    assert rc == 0
    assert np.linalg.norm(got.astype(np.float64) - want) <= 1e-6 * np.linalg.norm(want)
    rc, poly = oracle.moe_run(ex, shared, top, codes, scales, ids, routes, mode=1)
    assert rc == 0 and np.linalg.norm(poly.astype(np.float64) - want) <= 1e-6 * np.linalg.norm(want)
    # rejected arguments (src/rk_npu_moe_w8.cpp:586-595)
    bad = ids.copy(); bad[2, 0] = routed
    assert oracle.moe_run(ex, shared, top, codes, scales, bad, routes)[0] == 1
    neg = routes.copy(); neg[2, 1] = -0.5
    assert oracle.moe_run(ex, shared, top, codes, scales, ids, neg)[0] == 1
    zs = scales.copy(); zs[3] = 0
    assert oracle.moe_run(ex, shared, top, codes, zs, ids, routes)[0] == 1


def test_host_entry_points(lib):
    c = capi.MoeConfig()
    lib.rk_npu_moe_w8_config_init(C.byref(c), 1536, 512, 128, 1, 8, 256)
    # include/rk_npu_moe_w8.h:70-72: three cores, four threads, normal input, fp32 middle stage, one second
    assert (c.struct_size, c.weights.hidden, c.weights.intermediate, c.weights.routed_experts, c.weights.shared_expert) == \
        (C.sizeof(capi.MoeConfig), 1536, 512, 128, 1)
    assert (c.max_rows, c.top_k, c.npu_cores, c.cpu_threads, c.native_input, c.middle, c.timeout_ms) == (256, 8, 3, 4, 0, 0, 1000)
    assert C.sizeof(capi.MoeConfig) == 48 and C.sizeof(capi.MoeTimings) == 112 and C.sizeof(capi.MoeExpert) == 32
    lib.rk_npu_moe_w8_config_init(None, 64, 32, 1, 0, 1, 1)      # NULL is ignored
    assert lib.rk_npu_moe_w8_weights_device_bytes(None) == 0 and lib.rk_npu_moe_w8_workspace_device_bytes(None) == 0
    assert not lib.rk_npu_moe_w8_weights_create(None, C.byref(c.weights), None)
    assert not lib.rk_npu_moe_w8_workspace_create(None, C.byref(c))
    assert lib.rk_npu_moe_w8_run_f32(None, None, 1, None, None, None, None, None) == capi.RK_NPU_ERR_PARAM
    lib.rk_npu_moe_w8_weights_free(None)
    lib.rk_npu_moe_w8_workspace_free(None)
    # the int4 expert forms, the slot banks and their cache records validate their arguments like the int8 form
    for name in ("rk_npu_moe_quant_weights_create", "rk_npu_moe_quant_weights_create_full_k", "rk_npu_moe_w4_weights_create",
                 "rk_npu_moe_w4_slots_create"):
        assert not getattr(lib, name)(None, C.byref(c.weights), None)
    assert not lib.rk_npu_moe_quant_slots_create(None, C.byref(c.weights))
    assert not lib.rk_npu_moe_quant_workspace_create(None, C.byref(c)) and not lib.rk_npu_moe_w4_workspace_create(None, C.byref(c))
    assert lib.rk_npu_moe_quant_expert_blob_bytes(None) == 0
    assert lib.rk_npu_moe_quant_export_expert(None, 0, None, 0) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_moe_quant_import_expert(None, 0, None, 0) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_moe_quant_import_expert_timed(None, 0, None, 0, None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_moe_quant_swap_slots(None, 0, None, 0) == capi.RK_NPU_ERR_PARAM
