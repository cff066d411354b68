"""The search tuner on the GPU: search, save, reload without a device, build from the strategy, run.

Mirrors the reference's tuner tests (tests/test_w4a8_tune.cpp, tests/test_autotune_cpu.cpp:13-25): a search
returns validated strategies, a second cached call is a hit without device work, the file loads through the
load-only entry with an offline context, the tuned factories accept the strategy, results stay bit-exact,
and the workspace built from the fastest strategy is not slower than the library's own choice."""
import ctypes as C

import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from oracle.harness import make_activations, make_weights
from rknpu2_matmul_open_b200 import capi
from rknpu2_matmul_open_b200.capi import W4A8AutotuneConfig, W4A8StrategyEx

pytestmark = pytest.mark.gpu


def _time_graph(ws_handle, w, dA, dC, lib, torch, launches=20):
    stream = torch.cuda.Stream()
    def enqueue():
        for _ in range(launches):
            assert lib.rk_npu_b200_w4a8_enqueue_f16(ws_handle, w.handle, dA.data_ptr(), dC.data_ptr(), stream.cuda_stream) == 0
    with torch.cuda.stream(stream):
        enqueue()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        enqueue()
    best = 1e9
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        stream.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / launches)
    return best


@pytest.mark.parametrize("shape", [(8, 2048, 2048), (64, 4096, 1024)], ids=lambda s: "x".join(map(str, s)))
def test_search_save_reload_and_run(gpu, oracle, tmp_path, shape):
    import torch
    lib = capi.load()
    ctx, dom, _ = gpu
    M, K, N = shape
    B, sw = make_weights(K, N, seed=K + N)
    request = W4A8AutotuneConfig()
    lib.rk_npu_w4a8_autotune_config_init(C.byref(request), M, N, K)
    request.activation_type = capi.RK_NPU_W4A8_F16
    request.k_tile_multiplier = 1.0
    path = str(tmp_path / "tuned.tune").encode()
    fast, stable, hit = W4A8StrategyEx(), W4A8StrategyEx(), C.c_int(-1)
    Bp, sp = B.ctypes.data_as(C.c_void_p), sw.ctypes.data_as(C.c_void_p)
    assert lib.rk_npu_w4a8_autotune_cached_ex(ctx.handle, C.byref(request), Bp, sp, path, 0, C.byref(fast), C.byref(stable), C.byref(hit)) == 0
    assert hit.value == 0 and fast.base.total_us > 0 and stable.base.robust_us >= stable.base.total_us
    assert fast.base.tuning_revision == 5 and fast.base.config.M == M and fast.base.weights.config.K == K
    # a second call is answered from the file
    fast2, stable2 = W4A8StrategyEx(), W4A8StrategyEx()
    assert lib.rk_npu_w4a8_autotune_cached_ex(ctx.handle, C.byref(request), Bp, sp, path, 0, C.byref(fast2), C.byref(stable2), C.byref(hit)) == 0
    assert hit.value == 1 and bytes(fast2) == bytes(fast) and bytes(stable2) == bytes(stable)
    # and the file loads with no device behind the context: profile captured from a weight object, offline context
    w = rk.Weights(dom, B, sw, k_tile=fast.base.config.k_tile)
    profile = lib.rk_npu_w4a8_tuning_profile_from_weights(w.handle)
    offline = lib.rk_npu_b200_open_offline(lib.rk_npu_b200_driver_version(ctx.handle))
    fast3, stable3 = W4A8StrategyEx(), W4A8StrategyEx()
    assert lib.rk_npu_w4a8_autotune_cache_load_profile_ex(offline, C.byref(request), profile, path, C.byref(fast3), C.byref(stable3)) == 0
    assert bytes(fast3) == bytes(fast)
    lib.rk_npu_close(offline)
    lib.rk_npu_w4a8_tuning_profile_free(profile)
    # the factories accept the strategy; the tuned workspace computes the same bits
    wt = lib.rk_npu_w4a8_weights_create_tuned_ex(dom.handle, C.byref(fast), Bp, sp)
    tuned = lib.rk_npu_w4a8_workspace_create_tuned_ex(dom.handle, C.byref(fast))
    assert wt and tuned
    A = make_activations(M, K, seed=5, dtype="f16")
    out = np.zeros((M, N), np.uint16)
    assert lib.rk_npu_w4a8_run_f16(tuned, wt, A.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), None) == 0
    assert np.array_equal(out, oracle.linear(A, B, sw)[1])
    # not slower than the library's own choice (same weights, device tensors, one CUDA graph each)
    default = rk.Workspace(dom, rk.default_config(M, N, K, k_tile=fast.base.config.k_tile))
    dA = torch.from_numpy(A.view(np.int16)).cuda()
    dC = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    t_tuned = _time_graph(tuned, w, dA, dC, lib, torch)
    t_default = _time_graph(default.handle, w, dA, dC, lib, torch)
    assert t_tuned <= 1.15 * t_default + 0.3, (t_tuned, t_default, fast.base.config.pipeline, fast.base.config.m_tile, fast.base.config.n_tile)
    default.free()
    lib.rk_npu_w4a8_workspace_free(tuned)
    lib.rk_npu_w4a8_weights_free(wt)
    w.free()


def test_family_search_shares_one_tile(gpu, oracle):
    lib = capi.load()
    ctx, dom, _ = gpu
    K, N = 1024, 768
    B, sw = make_weights(K, N, seed=3)
    ms = (C.c_int * 3)(1, 8, 40)
    family = capi.W4A8FamilyConfig()
    lib.rk_npu_w4a8_family_config_init(C.byref(family), N, K, 3, ms)
    family.base.k_tile_multiplier = 1.0
    family.base.loops, family.base.repeats = 4, 3
    summary = capi.W4A8FamilySummary()
    strategies = (capi.W4A8Strategy * 3)()
    Bp, sp = B.ctypes.data_as(C.c_void_p), sw.ctypes.data_as(C.c_void_p)
    assert lib.rk_npu_w4a8_autotune_family(ctx.handle, C.byref(family), Bp, sp, C.byref(summary), strategies, None, None) == 0
    tiles = {s.config.k_tile for s in strategies}
    assert len(tiles) == 1 and summary.weights.config.k_tile in tiles and summary.weighted_total_us > 0
    assert [s.config.M for s in strategies] == [1, 8, 40]
    # bad requests: duplicate batch size, missing output array
    ms2 = (C.c_int * 2)(4, 4)
    lib.rk_npu_w4a8_family_config_init(C.byref(family), N, K, 2, ms2)
    assert lib.rk_npu_w4a8_autotune_family(ctx.handle, C.byref(family), Bp, sp, C.byref(summary), strategies, None, None) == capi.RK_NPU_ERR_PARAM
    lib.rk_npu_w4a8_family_config_init(C.byref(family), N, K, 3, ms)
    assert lib.rk_npu_w4a8_autotune_family(ctx.handle, C.byref(family), Bp, sp, C.byref(summary), None, None, None) == capi.RK_NPU_ERR_PARAM
