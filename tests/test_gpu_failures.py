"""Failure paths, every failure produced on the host or by a wait that is allowed to run out (nothing here
faults, traps or hangs a GPU).

Mirrors the reference's injections: allocation failure at every allocation index (tests/test_w4a8_low_cpu.cpp:
227-235: constructors return NULL and release what they had), and the timeout contract of a run
(include/rk_npu_w4a8.h:28: a device wait that exceeds timeout_ms ends the call with RK_NPU_ERR_SUBMIT and the
workspace stays usable)."""
import time

import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from oracle.harness import make_activations, make_weights
from rknpu2_matmul_open_b200 import capi

pytestmark = pytest.mark.gpu


def _stats(dom):
    s = dom.memory_stats()
    return s.live_bytes, s.creates - s.destroys


@pytest.mark.parametrize("shape", [(8, 1057, 385), (64, 1024, 512), (300, 640, 1000)], ids=lambda s: "x".join(map(str, s)))
def test_allocation_failure_at_every_index(gpu, oracle, shape):
    lib = capi.load()
    ctx, dom, _ = gpu
    M, K, N = shape
    B, sw = make_weights(K, N, seed=1)
    baseline = _stats(dom)
    try:
        # weights: fail the 1st, 2nd, ... allocation until creation goes through
        w, failures = None, 0
        for n in range(16):
            lib.rk_npu_b200_test_fail_allocation(n)
            try:
                w = rk.Weights(dom, B, sw)
                break
            except rk.W4A8Error:
                failures += 1
                assert _stats(dom) == baseline, f"weights: allocation {n} failed and something stayed allocated"
        lib.rk_npu_b200_test_fail_allocation(-1)
        assert w is not None and failures >= 2
        with_weights = _stats(dom)
        ws, failures = None, 0
        for n in range(32):
            lib.rk_npu_b200_test_fail_allocation(n)
            try:
                ws = rk.Workspace(dom, rk.default_config(M, N, K))
                break
            except rk.W4A8Error:
                failures += 1
                assert _stats(dom) == with_weights, f"workspace: allocation {n} failed and something stayed allocated"
        lib.rk_npu_b200_test_fail_allocation(-1)
        assert ws is not None and failures >= 5
    finally:
        lib.rk_npu_b200_test_fail_allocation(-1)
    # what was finally created works
    A = make_activations(M, K, seed=2, dtype="f32")
    out = np.zeros((M, N), np.float32)
    assert ws.run_f32(w, A, out) == 0
    assert np.array_equal(bits(out), bits(oracle.linear(A, B, sw)[1]))
    ws.free()
    w.free()
    assert _stats(dom) == baseline


def test_a_wait_that_runs_out_ends_the_call_with_submit_and_the_workspace_recovers(gpu, oracle):
    lib = capi.load()
    _, dom, _ = gpu
    M, K, N = 4, 2048, 1024
    B, sw = make_weights(K, N, seed=3)
    A = make_activations(M, K, seed=3, dtype="f16")
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K, timeout_ms=2))
    ref = oracle.linear(A, B, sw)[1]
    out = np.zeros((M, N), np.uint16)
    assert ws.run_f16(w, A, out) == 0 and np.array_equal(out, ref)
    assert lib.rk_npu_b200_w4a8_test_starve(ws.handle, 1) == 0
    t0 = time.perf_counter()
    assert ws.run_f16(w, A, out) == capi.RK_NPU_ERR_SUBMIT      # the bounded wait gave up after timeout_ms, the kernel returned
    assert time.perf_counter() - t0 < 1.0
    assert ws.run_f16(w, A, out) == capi.RK_NPU_ERR_SUBMIT      # and does so every time while the barrier is starved
    assert lib.rk_npu_b200_w4a8_test_starve(ws.handle, 0) == 0
    out[:] = 0
    assert ws.run_f16(w, A, out) == 0 and np.array_equal(out, ref)   # same workspace, clean run
    ws.free()
    w.free()


@pytest.mark.parametrize("M", [8, 24, 64, 300])
def test_a_recorded_device_error_is_reported_once_and_cleared(gpu, oracle, M):
    # the status word a kernel sets when a wait runs out, set from the host: every kernel family's host side
    # turns it into RK_NPU_ERR_SUBMIT, clears it (and its scratch), and the next run is exact
    lib = capi.load()
    _, dom, _ = gpu
    K, N = 1057, 513
    B, sw = make_weights(K, N, seed=4)
    A = make_activations(M, K, seed=4, dtype="f32")
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    assert lib.rk_npu_b200_w4a8_test_device_error(ws.handle) == 0
    assert ws.finish() == capi.RK_NPU_ERR_SUBMIT
    assert ws.finish() == 0
    out = np.zeros((M, N), np.float32)
    assert ws.run_f32(w, A, out) == 0
    assert np.array_equal(bits(out), bits(oracle.linear(A, B, sw)[1]))
    ws.free()
    w.free()
