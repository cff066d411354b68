"""The allocation-free linear (rk_npu_b200_w4a8_enqueue_f16_static) against the oracle and the
ordinary workspace entry point.

The entry point serves callers that must not allocate while they run -- an engine that fixed
its device memory budget at start-up, a plugin inside a latency-critical loop -- so it keeps
its scratch (activation codes, token scales, status) in an array inside the library image
instead of a workspace.  The array is shared by all calls and keeps old contents, so the
test calls it twice in a row, with different batch sizes and inputs, and expects each result
to equal (bit for bit, the tolerance of the other GPU tests) both the CPU oracle's linear and
what rk_npu_w4a8_run_f16 produces.  It also checks that sizes beyond the array are refused, that
nothing was allocated through the domain, and that the verdict of a call (a NaN row leaves the
output unwritten) can be read back without allocating.  The file sorts last so that a stop-at-first-failure run has
already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from oracle.harness import make_activations, make_weights
from rknpu2_matmul_open_b200 import capi

pytestmark = pytest.mark.gpu


def test_static_scratch_linear_matches_workspace_linear_twice(oracle):
    import torch
    lib = capi.load()
    bad, err = C.c_int(-1), C.c_int(-1)
    ctx = rk.Context("cuda:0")
    dom = ctx.domain(3)
    K, N = 1057, 385
    B, sw = make_weights(K, N, seed=77)
    w = rk.Weights(dom, B, sw)
    stream = torch.cuda.Stream()
    before = dom.memory_stats()
    results = []
    for call, M in enumerate((13, 5)):                      # second call is smaller: stale rows must not leak in
        A = make_activations(M, K, seed=100 + call, dtype="f16")
        dA = torch.from_numpy(A.view(np.int16)).cuda()
        dC = torch.full((M, N), 0x5555, dtype=torch.int16, device="cuda")
        torch.cuda.synchronize()
        rc = lib.rk_npu_b200_w4a8_enqueue_f16_static(w.handle, dA.data_ptr(), dC.data_ptr(), M, stream.cuda_stream)
        assert rc == 0
        stream.synchronize()
        assert lib.rk_npu_b200_w4a8_static_status(w.handle, C.byref(bad), C.byref(err)) == 0 and (bad.value, err.value) == (0, 0)
        results.append((A, dC.cpu().numpy().view(np.uint16)))
    after = dom.memory_stats()
    assert (after.creates, after.live_bytes) == (before.creates, before.live_bytes)   # nothing allocated on the way
    for A, got in results:
        M = A.shape[0]
        ws = rk.Workspace(dom, rk.default_config(M, N, K))
        ref = np.zeros((M, N), np.uint16)
        assert ws.run_f16(w, A, ref) == 0
        ws.free()
        rc, want, _, _ = oracle.linear(A, B, sw)
        assert rc == 0 and np.array_equal(got, want)        # the CPU oracle
        assert np.array_equal(got, ref)                     # and the workspace entry point
    # a NaN row: output untouched, and the verdict can be read back (still without allocating)
    before = dom.memory_stats()                             # (the comparison above created and freed workspaces)
    A = make_activations(4, K, seed=9, dtype="f16")
    A[2, 5] = 0x7E00
    dA = torch.from_numpy(A.view(np.int16)).cuda()
    dC = torch.full((4, N), 0x5555, dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()
    assert lib.rk_npu_b200_w4a8_enqueue_f16_static(w.handle, dA.data_ptr(), dC.data_ptr(), 4, stream.cuda_stream) == 0
    stream.synchronize()
    assert lib.rk_npu_b200_w4a8_static_status(w.handle, C.byref(bad), C.byref(err)) == capi.RK_NPU_ERR_PARAM
    assert (bad.value, err.value) == (1, 0) and int(dC.min()) == 0x5555 and int(dC.max()) == 0x5555
    after = dom.memory_stats()
    assert (after.creates, after.live_bytes) == (before.creates, before.live_bytes)
    # beyond the fixed array: refused with a clear code, output untouched
    dA = torch.zeros((33, K), dtype=torch.int16, device="cuda")
    dC = torch.full((33, N), 7, dtype=torch.int16, device="cuda")
    assert lib.rk_npu_b200_w4a8_enqueue_f16_static(w.handle, dA.data_ptr(), dC.data_ptr(), 33, stream.cuda_stream) == capi.RK_NPU_ERR_NOMEM
    assert lib.rk_npu_b200_w4a8_enqueue_f16_static(w.handle, None, dC.data_ptr(), 4, stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
    stream.synchronize()
    assert int(dC.min()) == 7 and int(dC.max()) == 7
    big_k = 65536 + 128
    wb = rk.Weights(dom, np.zeros((big_k, 32), np.int8), np.ones(32, np.float32))
    dA = torch.zeros((32, big_k), dtype=torch.int16, device="cuda")
    dC = torch.zeros((32, 32), dtype=torch.int16, device="cuda")
    assert lib.rk_npu_b200_w4a8_enqueue_f16_static(wb.handle, dA.data_ptr(), dC.data_ptr(), 32, stream.cuda_stream) == capi.RK_NPU_ERR_NOMEM
    assert lib.rk_npu_b200_w4a8_enqueue_f16_static(wb.handle, dA.data_ptr(), dC.data_ptr(), 16, stream.cuda_stream) == 0
    stream.synchronize()
    wb.free()
    w.free()
    dom.free()
    ctx.close()
