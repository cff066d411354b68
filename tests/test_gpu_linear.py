"""CUDA W4A8 linear through the C ABI against the oracle and the reference fixtures.
Integer accumulators and outputs are compared bit for bit (the bar: int32 exact,
fp16 within 1 ulp -- the observed difference is 0 ulp, so equality is asserted)."""
import ctypes as C
import threading

import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from oracle.harness import make_activations, make_weights, sample_columns
from rknpu2_matmul_open_b200 import capi

pytestmark = pytest.mark.gpu


def run_case(dom, oracle, A, B, sw, k_tile=480, split=0, **cfg_kw):
    M, K = A.shape
    N = B.shape[1]
    half = A.dtype == np.uint16
    w = rk.Weights(dom, B, sw, k_tile=k_tile)
    ws = rk.Workspace(dom, rk.default_config(M, N, K, k_tile=k_tile, **cfg_kw))
    if split:
        assert ws.set_schedule(0, split) == 0
    guard = 16
    out = np.full(M * N + 2 * guard, 0x5555 if half else -12345.0, np.uint16 if half else np.float32)
    body = out[guard:guard + M * N].reshape(M, N)
    rc = (ws.run_f16 if half else ws.run_f32)(w, A, body)
    acc = np.zeros((M, N), np.int32)
    rc_acc = ws.run_acc_i32(w, A, acc)
    ws.free()
    w.free()
    assert rc == 0 and rc_acc == 0
    assert np.all(out[:guard] == out[0]) and np.all(out[-guard:] == out[0]), "guard bytes touched"
    return body.copy(), acc


def test_reference_fixtures(gpu, golden_linear):
    _, dom, _ = gpu
    g = golden_linear
    for i in range(int(g["count"])):
        t = f"c{i}"
        kt = int(g[f"{t}_shape"][3])
        for A, ref_out, ref_acc in ((g[f"{t}_A32"], g[f"{t}_out32"], g[f"{t}_acc32"]),
                                    (g[f"{t}_A16"], g[f"{t}_out16"], g[f"{t}_acc16"])):
            out, acc = run_case(dom, None, A, g[f"{t}_B"], g[f"{t}_sw"], k_tile=kt)
            assert np.array_equal(acc, ref_acc), f"fixture {i}: int32"
            assert np.array_equal(bits(out), bits(ref_out)), f"fixture {i}: output"


# tail shapes from the reference's own tests (board tests, chain tests, low-CPU tests)
SHAPES = [(1, 1, 1), (3, 33, 65), (5, 1025, 129), (7, 513, 257), (65, 513, 1025), (65, 1441, 1025), (65, 1921, 1025),
          (1, 1057, 193), (2, 1057, 193), (4, 1057, 193), (8, 1057, 193), (33, 1057, 257), (17, 480, 64), (21, 97, 65),
          (21, 224, 65), (16, 513, 193), (17, 513, 193), (19, 1025, 257), (129, 2401, 1025), (257, 993, 257),
          (129, 2049, 257), (21, 992, 65)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_tail_shapes_both_dtypes(gpu, oracle, shape):
    _, dom, _ = gpu
    M, K, N = shape
    B, sw = make_weights(K, N, seed=K + N)
    for dtype in ("f32", "f16"):
        A = make_activations(M, K, seed=M + K, dtype=dtype)
        if M > 1:
            A[0, :] = 0          # an all-zero row must give scale 1 and exact zeros
        out, acc = run_case(dom, oracle, A, B, sw)
        rc, ref, ref_acc, _ = oracle.linear(A, B, sw)
        assert rc == 0
        assert np.array_equal(acc, ref_acc)
        assert np.array_equal(bits(out), bits(ref))
        if M > 1:
            assert not out[0].any()


def test_extreme_codes_large_sums_and_fp16_overflow(gpu, oracle):
    # +-127 activations x {-8, 7} weights: sums beyond 2^24 and fp16 results that overflow to inf
    _, dom, _ = gpu
    for (M, K, N) in [(2, 480, 64), (5, 1025, 129), (2, 20003, 65), (1, 20003, 193)]:
        B = np.where((np.arange(K * N) % N % 2).reshape(K, N) == 1, 7, -8).astype(np.int8)
        if N == 193:
            B[:] = -8
        sw = np.ldexp(np.float32(1), -(np.arange(N) % 6 + 6)).astype(np.float32)
        A32 = np.where((np.arange(M) % 2)[:, None] == 1, np.float32(127), np.float32(-127)) * np.ones((1, K), np.float32)
        for A in (A32, oracle.float_to_half(A32)):
            out, acc = run_case(dom, oracle, A, B, sw)
            rc, ref, ref_acc, _ = oracle.linear(A, B, sw)
            assert np.array_equal(acc, ref_acc) and np.array_equal(bits(out), bits(ref))
    assert np.abs(ref_acc).max() > 2 ** 24


@pytest.mark.parametrize("split", [1, 2, 3, 4, 5, 6, 7, 8])
def test_split_k_clusters_are_exact(gpu, oracle, split, monkeypatch):
    _, dom, _ = gpu
    shapes = [(8, 2048, 512), (16, 1153, 257), (32, 2048, 384), (8, 2048 * split, 256)]
    if split in (1, 2, 4, 8):
        shapes.append((40, 640, 130))        # larger batch: quantise kernel + split-K GEMM kernel
        shapes.append((16, 2048, 384))       # default schedule above 8 tokens: quantise kernel + cluster split-K ring
    else:
        monkeypatch.setenv("RK_NPU_B200_VARIANT", "3")   # odd cluster sizes exist only in the single-kernel path
    for (M, K, N) in shapes:
        B, sw = make_weights(K, N, seed=split)
        A = make_activations(M, K, seed=split, dtype="f16")
        out, acc = run_case(dom, oracle, A, B, sw, split=split)
        rc, ref, ref_acc, _ = oracle.linear(A, B, sw)
        assert np.array_equal(acc, ref_acc) and np.array_equal(bits(out), bits(ref))
    if split in (1, 2, 4, 8):
        # the same cluster sizes through the single-kernel path at 16 and 32 tokens
        monkeypatch.setenv("RK_NPU_B200_VARIANT", "3")
        for (M, K, N) in [(16, 1153, 257), (32, 2048, 384)]:
            B, sw = make_weights(K, N, seed=split)
            A = make_activations(M, K, seed=split, dtype="f16")
            out, acc = run_case(dom, oracle, A, B, sw, split=split)
            rc, ref, ref_acc, _ = oracle.linear(A, B, sw)
            assert np.array_equal(acc, ref_acc) and np.array_equal(bits(out), bits(ref))


def test_scheduling_hints_do_not_change_results(gpu, oracle):
    # tiles, core masks, pipelines, thread counts, layouts and reduce backends are hints here
    ctx, dom, _ = gpu
    M, K, N = 37, 1441, 449
    B, sw = make_weights(K, N, seed=21)
    A = make_activations(M, K, seed=21, dtype="f32")
    rc, ref, _, _ = oracle.linear(A, B, sw)
    w = rk.Weights(dom, B, sw, k_tile=256)
    for kw in (dict(m_tile=3, n_tile=128), dict(m_tile=64, n_tile=1408, npu_core_mask=7, cpu_threads=4),
               dict(pipeline=0), dict(pipeline=2, npu_core_mask=3)):
        for options in (None, capi.W4A8Options(C.sizeof(capi.W4A8Options), 0, 1)):
            ws = rk.Workspace(dom, rk.default_config(M, N, K, k_tile=256, **kw), options if kw.get("pipeline") != 2 else None)
            out = np.zeros((M, N), np.float32)
            assert ws.run_f32(w, A, out) == 0
            assert np.array_equal(bits(out), bits(ref))
            ws.free()
    o = capi.W4A8Options(C.sizeof(capi.W4A8Options), 1, 0)
    ws = rk.Workspace(dom, rk.default_config(M, N, K, k_tile=256, m_tile=32), o)
    out = np.zeros((M, N), np.float32)
    assert ws.run_f32(w, A, out) == 0 and np.array_equal(bits(out), bits(ref))
    ws.free()
    w.free()


def test_quantized_codes_and_scales(gpu, oracle):
    _, dom, _ = gpu
    M, K, N = 5, 533, 64
    a = np.zeros((M, K), np.float32)
    for m in range(1, M):
        a[m] = np.ldexp((np.arange(K) % 255 - 127).astype(np.float32), m - 3)
        a[m, K - 1] = np.ldexp(np.float32(254), m - 3)   # the row maximum sits in the last element
    a[1] = (np.arange(K) % 255 - 127).astype(np.float32)
    a[1, 1:5] = [.5, -.5, 1.5, -1.5]                     # exact ties round away from zero
    B, sw = make_weights(K, N, seed=1)
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    for A in (a, oracle.float_to_half(a)):
        out = np.zeros((M, N), A.dtype)
        assert (ws.run_f16 if A.dtype == np.uint16 else ws.run_f32)(w, A, out) == 0
        assert ws.run_acc_i32(w, A, np.zeros((M, N), np.int32)) == 0
        rc, s, q = ws.last_quant()
        _, so, inv = oracle.scales(A)
        assert rc == 0 and np.array_equal(bits(s), bits(so)) and np.array_equal(q, oracle.quantize(A, inv))
        assert s[0] == 1 and list(q[1, 1:5]) == [1, -1, 2, -2]
    tiny = np.full((M, K), 1e-45, np.float32)
    out = np.zeros((M, N), np.float32)
    assert ws.run_f32(w, tiny, out) == 0
    assert np.all(ws.last_quant()[1] == np.float32(1.17549435e-38))
    ws.free()
    w.free()


def test_shared_weights_rebinding_and_domains(gpu, oracle):
    # one immutable weight object serves any M and both dtypes; a workspace can be rebound;
    # objects of another domain are refused before any work (tests/test_w4a8.cpp:125-162)
    ctx, dom, other = gpu
    K, N = 513, 193
    B1, B2 = np.full((K, N), 3, np.int8), np.full((K, N), -2, np.int8)
    s1, s2 = np.full(N, .01, np.float32), np.full(N, .003, np.float32)
    w1, w2 = rk.Weights(dom, B1, s1, k_tile=256), rk.Weights(dom, B2, s2, k_tile=256)
    foreign = rk.Weights(other, B1, s1, k_tile=256)
    for M in (1, 5, 65):
        ws = rk.Workspace(dom, rk.default_config(M, N, K, k_tile=256, m_tile=16, n_tile=64, npu_core_mask=7))
        a = (np.arange(M * K) % 255 - 127).astype(np.float32).reshape(M, K)
        for w, B, s, half in ((w1, B1, s1, False), (w2, B2, s2, True), (w1, B1, s1, True)):
            A = oracle.float_to_half(a) if half else a
            out = np.zeros((M, N), A.dtype)
            assert (ws.run_f16 if half else ws.run_f32)(w, A, out) == 0
            assert np.array_equal(bits(out), bits(oracle.linear(A, B, s)[1]))
        assert ws.run_f32(foreign, a, np.zeros((M, N), np.float32)) == capi.RK_NPU_ERR_DOMAIN
        ws.free()
    for w in (w1, w2, foreign):
        w.free()


def test_argument_errors(gpu, oracle):
    ctx, dom, _ = gpu
    lib = capi.load()
    K, N, M = 256, 128, 4
    B, sw = make_weights(K, N, seed=4)
    # invalid weights -> NULL
    for bad_scale in (0.0, np.inf, -1.0, np.nan):
        s = sw.copy()
        s[1] = bad_scale
        with pytest.raises(rk.W4A8Error):
            rk.Weights(dom, B, s)
    Bb = B.copy()
    Bb[0, 0] = 8
    with pytest.raises(rk.W4A8Error):
        rk.Weights(dom, Bb, sw)
    Bb[0, 0] = -9
    with pytest.raises(rk.W4A8Error):
        rk.Weights(dom, Bb, sw)
    with pytest.raises(rk.W4A8Error):                      # explicit tile above 480 must be certified
        rk.Weights(dom, np.full((2048, 64), -8, np.int8), np.ones(64, np.float32), k_tile=512)
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    A = make_activations(M, K, seed=4, dtype="f32")
    out = np.zeros((M, N), np.float32)
    t = capi.W4A8Timings()
    assert lib.rk_npu_w4a8_run_f32(None, w.handle, A.ctypes.data, out.ctypes.data, None) == -3
    assert lib.rk_npu_w4a8_run_f32(ws.handle, None, A.ctypes.data, out.ctypes.data, None) == -3
    assert lib.rk_npu_w4a8_run_f32(ws.handle, w.handle, None, out.ctypes.data, None) == -3
    assert lib.rk_npu_w4a8_run_f32(ws.handle, w.handle, A.ctypes.data, A.ctypes.data, None) == -3   # aliasing
    w_other = rk.Weights(dom, B, sw, k_tile=256)
    assert ws.run_f32(w_other, A, out) == -3               # k_tile is part of the weight key
    w_other.free()
    # NaN / Inf activations: PARAM, no GEMM time, and the workspace keeps working afterwards
    for bad in (np.nan, np.inf, -np.inf):
        Abad = A.copy()
        Abad[M - 1, K - 1] = bad
        assert ws.run_f32(w, Abad, out, t) == -3 and t.submit_us == 0
    h = oracle.float_to_half(A)
    h[0, 0] = 0xfc00
    assert ws.run_f16(w, h, np.zeros((M, N), np.uint16), t) == -3 and t.submit_us == 0
    assert ws.run_f32(w, A, out, t) == 0 and t.submit_us > 0 and t.total_us > 0
    assert np.array_equal(bits(out), bits(oracle.linear(A, B, sw)[1]))
    # workspace geometry errors -> NULL
    for kw in (dict(m_tile=0), dict(k_tile=0), dict(n_tile=32), dict(cpu_threads=5), dict(npu_core_mask=5)):
        with pytest.raises(rk.W4A8Error):
            rk.Workspace(dom, rk.default_config(M, N, K, **kw))
    ws.free()
    w.free()


def test_auto_k_tile_and_weight_info(gpu, oracle, monkeypatch):
    ctx, dom, _ = gpu
    monkeypatch.delenv("RK_NPU_W4A8_K_TILE_MULTIPLIER", raising=False)
    K, N = 2048, 64
    for fill, expected in ((-8, 480), (4, 1024), (0, 2048)):
        w = rk.Weights(dom, np.full((K, N), fill, np.int8), np.ones(N, np.float32), k_tile=0)
        info = w.info()
        assert (info.config.K, info.config.N, info.config.k_tile, info.safe_k_tile, info.multiplier, info.bound_relaxed) == \
            (K, N, expected, expected, 1.0, 0)
        w.free()
    monkeypatch.setenv("RK_NPU_W4A8_K_TILE_MULTIPLIER", "1.5")
    w = rk.Weights(dom, np.full((K, N), -8, np.int8), np.ones(N, np.float32), k_tile=0)
    info = w.info()
    assert info.config.k_tile == 704 and info.safe_k_tile == 480 and info.multiplier == 1.5 and info.bound_relaxed == 1
    # An uncertified tile saturates INT16 partials on the original device; the int32
    # accumulation here stays exact, so the result still equals the integer formula.
    M = 2
    A = np.full((M, K), 127.0, np.float32)
    ws = rk.Workspace(dom, rk.default_config(M, N, K, k_tile=704))
    out = np.zeros((M, N), np.float32)
    assert ws.run_f32(w, A, out) == 0
    assert np.array_equal(bits(out), bits(oracle.linear(A, np.full((K, N), -8, np.int8), np.ones(N, np.float32))[1]))
    ws.free()
    w.free()
    for bad in ("0.5", "abc", "1.5x", "inf", ""):
        monkeypatch.setenv("RK_NPU_W4A8_K_TILE_MULTIPLIER", bad)
        with pytest.raises(rk.W4A8Error):
            rk.Weights(dom, np.zeros((K, N), np.int8), np.ones(N, np.float32), k_tile=0)


def test_busy_workspace(gpu, oracle):
    ctx, dom, _ = gpu
    M, K, N = 32, 8192, 4096
    B, sw = make_weights(K, N, seed=8)
    A = make_activations(M, K, seed=8, dtype="f32")
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    outs = [np.zeros((M, N), np.float32) for _ in range(2)]
    codes = []
    barrier = threading.Barrier(2)

    def worker(i):
        barrier.wait()
        for _ in range(50):
            codes.append(ws.run_f32(w, A, outs[i]))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert set(codes) <= {0, capi.RK_NPU_ERR_BUSY} and codes.count(0) >= 50
    ws.free()
    w.free()


def test_device_pointers_and_enqueue(gpu, oracle):
    import torch
    ctx, dom, _ = gpu
    M, K, N = 8, 4096, 4096
    B, sw = make_weights(K, N, seed=2)
    A = make_activations(M, K, seed=2, dtype="f16")
    rc, ref, _, _ = oracle.linear(A, B, sw)
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    dA = torch.from_numpy(A.view(np.int16)).cuda()
    dC = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    assert ws.run_f16(w, dA, dC) == 0                      # blocking call, device tensors
    assert np.array_equal(dC.cpu().numpy().view(np.uint16), ref)
    dC.zero_()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            assert ws.enqueue_f16(w, dA, dC, stream.cuda_stream) == 0
    stream.synchronize()
    assert ws.finish() == 0
    assert np.array_equal(dC.cpu().numpy().view(np.uint16), ref)
    bad = dA.clone()
    bad[3, 7] = 0x7c00                                      # +inf
    assert ws.enqueue_f16(w, bad, dC, stream.cuda_stream) == 0
    stream.synchronize()
    assert ws.finish() == capi.RK_NPU_ERR_PARAM
    assert ws.enqueue_f16(w, dA, dC, stream.cuda_stream) == 0
    stream.synchronize()
    assert ws.finish() == 0
    ws.free()
    w.free()


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (4, 1057, 385), (8, 4096, 4096), (8, 2048, 513), (24, 1057, 385)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_page_locked_host_tensors(gpu, oracle, shape, dtype):
    # small batches write a page-locked result tensor from the kernel itself and report into page-locked memory:
    # same numbers, same verdicts, nothing outside the result touched
    import torch
    lib = capi.load()
    _, dom, _ = gpu
    M, K, N = shape
    half = dtype == "f16"
    B, sw = make_weights(K, N, seed=11)
    A = make_activations(M, K, seed=11, dtype=dtype)
    ref = oracle.linear(A, B, sw)[1]
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K, timeout_ms=2))
    hA = torch.from_numpy(A.view(np.int16) if half else A).pin_memory()
    guard = 64
    flat = torch.full((M * N + 2 * guard,), 0x5555 if half else -7, dtype=torch.int16 if half else torch.float32).pin_memory()
    hC = flat[guard:guard + M * N].view(M, N)
    run = ws.run_f16 if half else ws.run_f32
    for _ in range(2):
        hC.zero_()
        assert run(w, hA, hC) == 0
        assert np.array_equal(bits(hC.numpy().view(np.uint16) if half else hC.numpy()), bits(ref))
    assert torch.all(flat[:guard] == flat[0]) and torch.all(flat[-guard:] == flat[0]), "guard elements touched"
    bad = hA.clone().pin_memory()
    bad[M - 1, K - 1] = 0x7c00 if half else float("nan")
    assert run(w, bad, hC) == capi.RK_NPU_ERR_PARAM
    assert run(w, hA, hC) == 0
    if ws.schedule()[0] == 5:
        assert lib.rk_npu_b200_w4a8_test_starve(ws.handle, 1) == 0
        assert run(w, hA, hC) == capi.RK_NPU_ERR_SUBMIT      # a bounded wait ran out; reported through the page-locked block
        assert lib.rk_npu_b200_w4a8_test_starve(ws.handle, 0) == 0
    hC.zero_()
    assert run(w, hA, hC) == 0
    assert np.array_equal(bits(hC.numpy().view(np.uint16) if half else hC.numpy()), bits(ref))
    ws.free()
    w.free()


def test_full_size_decode_sampled(gpu, oracle):
    # the benchmark's decode shapes at full size: 17 sampled columns x all rows (the reference's
    # own sampling for large shapes) plus linearity in the weights scale as a whole-output property
    ctx, dom, _ = gpu
    for (M, K, N) in [(1, 4096, 4096), (8, 4096, 11008), (8, 11008, 4096)]:
        B, sw = make_weights(K, N, seed=N)
        A = make_activations(M, K, seed=N, dtype="f16")
        w = rk.Weights(dom, B, sw)
        ws = rk.Workspace(dom, rk.default_config(M, N, K))
        acc = np.zeros((M, N), np.int32)
        assert ws.run_acc_i32(w, A, acc) == 0
        cols = sample_columns(N)
        _, _, inv = oracle.scales(A)
        assert np.array_equal(acc[:, cols], oracle.gemm_i32_columns(oracle.quantize(A, inv), B, cols))
        out = np.zeros((M, N), np.uint16)
        assert ws.run_f16(w, A, out) == 0
        _, s, _ = oracle.scales(A)
        assert np.array_equal(out, oracle.dequant(acc, s, sw, True))   # epilogue exact over the whole output
        w2 = rk.Weights(dom, B, sw * np.float32(2))
        out2 = np.zeros((M, N), np.uint16)
        assert ws.run_f16(w2, A, out2) == 0
        f1, f2 = oracle.half_to_float(out), oracle.half_to_float(out2)
        finite = np.isfinite(f2) & (np.abs(f1) > 1e-4)
        assert np.array_equal(f2[finite], (f1 * 2)[finite])            # power-of-two scaling is exact
        for x in (ws, w, w2):
            x.free()


# Every schedule the library can pick for a small batch (1: quantise + mma.sync ring, 3: single fused
# kernel, 4: quantise + persistent tcgen05 streaming kernel with its cross-CTA integer fix-up) has to
# give the same bits; the shapes make the streaming kernel split tiles between CTAs in the middle of K.
@pytest.mark.parametrize("variant", [1, 3, 4])
@pytest.mark.parametrize("shape", [(1, 4096, 4096), (8, 2304, 1000), (13, 1441, 385), (16, 5000, 300), (32, 1100, 2049),
                                   (27, 8192, 512)], ids=lambda s: "x".join(map(str, s)))
def test_small_batch_schedules_agree(gpu, oracle, monkeypatch, variant, shape):
    _, dom, _ = gpu
    M, K, N = shape
    monkeypatch.setenv("RK_NPU_B200_VARIANT", str(variant))
    B, sw = make_weights(K, N, seed=3 * K + N)
    for dtype in ("f16", "f32"):
        A = make_activations(M, K, seed=M + K, dtype=dtype)
        out, acc = run_case(dom, oracle, A, B, sw)
        out2, _ = run_case(dom, oracle, A, B, sw)            # the scratch buffers must come back clean
        rc, ref, ref_acc, _ = oracle.linear(A, B, sw)
        assert rc == 0
        assert np.array_equal(acc, ref_acc)
        assert np.array_equal(bits(out), bits(ref))
        assert np.array_equal(bits(out2), bits(ref))


def test_streaming_schedule_reuses_one_workspace(gpu, oracle, monkeypatch):
    # many launches through ONE workspace of the streaming schedule: partial-sum slots and
    # counters are handed back zeroed by the CTA that finishes each tile
    _, dom, _ = gpu
    monkeypatch.setenv("RK_NPU_B200_VARIANT", "4")
    M, K, N = 5, 3000, 1500
    B, sw = make_weights(K, N, seed=9)
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    for rep in range(6):
        A = make_activations(M, K, seed=rep, dtype="f32")
        out = np.zeros((M, N), np.float32)
        assert ws.run_f32(w, A, out) == 0
        rc, ref, _, _ = oracle.linear(A, B, sw)
        assert rc == 0 and np.array_equal(bits(out), bits(ref)), rep
    bad = make_activations(M, K, seed=1, dtype="f32")
    bad[2, 17] = np.nan
    assert ws.run_f32(w, bad, out) == capi.RK_NPU_ERR_PARAM   # rejected rows leave the scratch untouched
    A = make_activations(M, K, seed=77, dtype="f32")
    assert ws.run_f32(w, A, out) == 0
    assert np.array_equal(bits(out), bits(oracle.linear(A, B, sw)[1]))
    ws.free()
    w.free()


# 33..128 tokens: the mma.sync ring in 32-token chunks (1), the per-tile tcgen05 kernel (2) and the persistent
# streaming kernel (4, token tiles of 64 and 128, partial tiles combined across CTAs) against the oracle,
# plain and ragged shapes
@pytest.mark.parametrize("variant", [1, 2, 4])
@pytest.mark.parametrize("shape", [(33, 1057, 257), (64, 4096, 1024), (100, 2304, 385), (128, 11008, 512), (65, 8192, 130)],
                         ids=lambda s: "x".join(map(str, s)))
def test_mid_batch_schedules_agree(gpu, oracle, monkeypatch, variant, shape):
    _, dom, _ = gpu
    M, K, N = shape
    monkeypatch.setenv("RK_NPU_B200_VARIANT", str(variant))
    B, sw = make_weights(K, N, seed=K + 7 * N)
    for dtype in ("f16", "f32"):
        A = make_activations(M, K, seed=M + K, dtype=dtype)
        out, acc = run_case(dom, oracle, A, B, sw)
        out2, _ = run_case(dom, oracle, A, B, sw)
        rc, ref, ref_acc, _ = oracle.linear(A, B, sw)
        assert rc == 0
        assert np.array_equal(acc, ref_acc)
        assert np.array_equal(bits(out), bits(ref))
        assert np.array_equal(bits(out2), bits(ref))


# The single-kernel path with two column tiles per CTA (chosen by itself for launches that would fill more than
# half of the GPU's shared memory; forced here on small shapes): even, odd and single tile counts, every
# cluster size, both input types, a rejected input (nothing may be left waiting for the second tile).
@pytest.mark.parametrize("shape", [(1, 4096, 4096), (8, 2304, 1000), (13, 1441, 385), (8, 1057, 257), (16, 640, 129),
                                   (32, 1100, 2049), (5, 513, 64)], ids=lambda s: "x".join(map(str, s)))
def test_single_kernel_two_tiles_per_cta(gpu, oracle, monkeypatch, shape):
    _, dom, _ = gpu
    M, K, N = shape
    monkeypatch.setenv("RK_NPU_B200_VARIANT", "3")
    monkeypatch.setenv("RK_NPU_B200_TILES_PER_CTA", "2")
    B, sw = make_weights(K, N, seed=5 * K + N)
    for dtype in ("f16", "f32"):
        A = make_activations(M, K, seed=M + K, dtype=dtype)
        rc, ref, ref_acc, _ = oracle.linear(A, B, sw)
        assert rc == 0
        for split in (0, 1, 2, 3, 8):
            kb = (K + 127) // 128
            if split and (kb < split or (kb + split - 1) // split > 16):     # at most 16 k-blocks per CTA
                continue
            out, acc = run_case(dom, oracle, A, B, sw, split=split)
            assert np.array_equal(acc, ref_acc)
            assert np.array_equal(bits(out), bits(ref))
    # NaN input: PARAM without a timeout, then the same workspace computes again
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    A = make_activations(M, K, seed=1, dtype="f32")
    bad = A.copy()
    bad[M - 1, K // 2] = np.nan
    out = np.zeros((M, N), np.float32)
    t = capi.W4A8Timings()
    assert ws.run_f32(w, bad, out, t) == capi.RK_NPU_ERR_PARAM
    assert t.total_us < 100e3          # far below the 500 ms a bounded wait would take to give up
    assert ws.run_f32(w, A, out) == 0
    assert np.array_equal(bits(out), bits(oracle.linear(A, B, sw)[1]))
    ws.free()
    w.free()
