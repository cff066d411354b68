"""CUDA routed experts through the C ABI against the oracle: outputs bit for bit (the oracle evaluates the middle
stage with the polynomial of the original's production target, as the kernels do), every rejection of the
original's run call and the untouched output behind it, rebinding, empty routes.  Cases follow the original's board
test tests/test_moe_w8.cpp (1, 5, 128, 256 rows; duplicate ids; zero coefficients; experts nobody selects; a shared
expert; nearest-even fp32 input; foreign domain)."""
import ctypes as C

import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from rknpu2_matmul_open_b200 import capi, moe

pytestmark = pytest.mark.gpu


def make_experts(H, I, E, seed, small=False):
    rng = np.random.default_rng(seed)
    lo, hi = (-3, 4) if small else (-127, 128)
    ex = dict(gate_up=rng.integers(lo, hi, size=(E, H, 2 * I), dtype=np.int8),
              gate_up_scales=rng.uniform(2e-4, 6e-4, size=(E, 2 * I)).astype(np.float32) * (16 if small else 1),
              down=rng.integers(lo, hi, size=(E, I, H), dtype=np.int8),
              down_scales=rng.uniform(1e-3, 3e-3, size=(E, H)).astype(np.float32))
    if not small:
        ex["gate_up"][rng.random(ex["gate_up"].shape) < 0.01] = -128
    return ex


def make_routes(rows, routed, top, seed):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, routed, size=(rows, top)).astype(np.int32)
    routes = rng.uniform(0.05, 0.95, size=(rows, top)).astype(np.float32)
    ids[0, :] = ids[0, 0]                     # duplicates: summed in slot order
    routes[rows // 2, top - 1] = 0            # a zero coefficient leaves the route out
    return ids, routes


SHAPES = [  # hidden, intermediate, routed, shared, top_k, max_rows, rows of the runs
    (64, 32, 3, 1, 2, 256, (1, 5, 128, 256, 1)),          # the board test's geometry
    (1536, 512, 16, 1, 8, 40, (33, 1, 17)),               # the documented envelope's corner
    (2048, 512, 8, 0, 2, 16, (7, 16)),
    (96, 64, 128, 1, 8, 64, (64,)),                       # many experts, most of them idle
    (8128, 64, 3, 1, 2, 8, (5,)),                         # widest hidden size the original's API mentions
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s[:6])))
def test_runs_equal_the_oracle(gpu, oracle, shape):
    _, dom, _ = gpu
    H, I, routed, shared, top, max_rows, row_counts = shape
    ex_a, ex_b = make_experts(H, I, routed + shared, seed=1), make_experts(H, I, routed + shared, seed=2)
    wa = moe.MoeWeights(dom, shared_expert=shared, **ex_a)
    wb = moe.MoeWeights(dom, shared_expert=shared, **ex_b)
    ws = moe.MoeWorkspace(dom, moe.default_config(H, I, routed, shared, top, max_rows))
    assert wa.device_bytes() >= (routed + shared) * 3 * H * I and ws.device_bytes() > 0
    for n, rows in enumerate(row_counts):
        rng = np.random.default_rng(10 + n)
        codes = rng.integers(-127, 128, size=(rows, H), dtype=np.int8)
        scales = rng.uniform(0.01, 0.05, size=rows).astype(np.float32)
        ids, routes = make_routes(rows, routed, top, seed=20 + n)
        guard = 32
        flat = np.full(rows * H + 2 * guard, -12345.0, np.float32)
        out = flat[guard:guard + rows * H].reshape(rows, H)
        for w, ex in ((wa, ex_a), (wb, ex_b), (wa, ex_a)):            # immutable weights are rebound per run
            rc_ref, ref = oracle.moe_run(ex, shared, top, codes, scales, ids, routes, mode=1)
            t = capi.MoeTimings()
            assert rc_ref == 0 and ws.run_quantized(w, codes, scales, ids, routes, out, t) == 0
            assert np.array_equal(bits(out), bits(ref)), f"rows={rows}"
            assert t.total_us > 0 and t.gemm_tasks > 0 and t.gather_tasks == t.middle_tasks > 0
            first = out.copy()
            assert ws.run_quantized(w, codes, scales, ids, routes, out) == 0 and np.array_equal(bits(out), bits(first))
        assert np.all(flat[:guard] == -12345.0) and np.all(flat[-guard:] == -12345.0), "guard values touched"
        # fp32 rows are quantised with nearest-even rounding: same result as the pre-quantised entry
        x = (rng.standard_normal((rows, H)) * 2).astype(np.float32)
        x[0, :8] = [127, -127, .5, 1.5, 2.5, -.5, -1.5, -2.5]
        if rows > 2:
            x[2] = 0                                                  # a zero row: scale 1, codes 0
        rc_q, q, s = oracle.moe_quantize_rows(x)
        rc_ref, ref = oracle.moe_run(ex_a, shared, top, q, s, ids, routes, mode=1)
        assert rc_q == 0 and rc_ref == 0
        assert ws.run_f32(wa, x, ids, routes, out) == 0
        assert np.array_equal(bits(out), bits(ref))
    ws.free(); wa.free(); wb.free()


def test_rejections_leave_the_output_alone(gpu, oracle):
    ctx, dom, other = gpu
    H, I, routed, shared, top, rows = 64, 32, 3, 1, 2, 5
    ex = make_experts(H, I, routed + shared, seed=3, small=True)
    w = moe.MoeWeights(dom, shared_expert=shared, **ex)
    ws = moe.MoeWorkspace(dom, moe.default_config(H, I, routed, shared, top, 16))
    rng = np.random.default_rng(4)
    codes = rng.integers(-127, 128, size=(rows, H), dtype=np.int8)
    scales = np.full(rows, 0.03125, np.float32)
    ids, routes = make_routes(rows, routed, top, seed=5)
    out = np.zeros((rows, H), np.float32)
    assert ws.run_quantized(w, codes, scales, ids, routes, out) == 0
    saved = out.copy()
    P = capi.RK_NPU_ERR_PARAM

    def rejected(rc):
        assert rc == P and np.array_equal(bits(out), bits(saved)), "a rejected call wrote the output"

    bad = ids.copy(); bad[0, 0] = routed                   # the shared expert's index is not a route
    rejected(ws.run_quantized(w, codes, scales, bad, routes, out))
    bad[0, 0] = -1
    rejected(ws.run_quantized(w, codes, scales, bad, routes, out))
    for value in (-0.25, np.nan, np.inf):
        r = routes.copy(); r[1, 1] = value
        rejected(ws.run_quantized(w, codes, scales, ids, r, out))
    for value in (0.0, -1.0, np.nan, np.inf):
        s = scales.copy(); s[2] = value
        rejected(ws.run_quantized(w, codes, s, ids, routes, out))
    x = rng.standard_normal((rows, H)).astype(np.float32)
    for value in (np.nan, np.inf, -np.inf):
        y = x.copy(); y[3, 7] = value
        rejected(ws.run_f32(w, y, ids, routes, out))
    tiny = np.zeros((rows, H), np.float32); tiny[0, 0] = 1e-45   # the row's scale underflows: its reciprocal is not finite
    rejected(ws.run_f32(w, tiny, ids, routes, out))
    big = np.zeros((17, H), np.float32)
    rejected(ws.lib.rk_npu_moe_w8_run_f32(ws.handle, w.handle, 17, big.ctypes.data, ids.ctypes.data, routes.ctypes.data,
                                          out.ctypes.data, None))                      # more rows than the workspace was made for
    rejected(ws.lib.rk_npu_moe_w8_run_f32(ws.handle, w.handle, 0, x.ctypes.data, ids.ctypes.data, routes.ctypes.data,
                                          out.ctypes.data, None))
    assert ws.run_f32(w, x, ids, routes, x) == P                                        # input and output overlap
    as_out = np.zeros((rows, H), np.float32)
    assert ws.lib.rk_npu_moe_w8_run_f32(ws.handle, w.handle, rows, x.ctypes.data, ids.ctypes.data, as_out.ctypes.data,
                                        as_out.ctypes.data, None) == P                 # coefficients and output overlap
    for missing in range(5):
        args = [x.ctypes.data, ids.ctypes.data, routes.ctypes.data, out.ctypes.data]
        if missing < 4:
            args[missing] = None
            rejected(ws.lib.rk_npu_moe_w8_run_f32(ws.handle, w.handle, rows, *args, None))
        else:
            rejected(ws.lib.rk_npu_moe_w8_run_quantized(ws.handle, w.handle, rows, codes.ctypes.data, None, ids.ctypes.data,
                                                        routes.ctypes.data, out.ctypes.data, None))
    # weights of another geometry, of another domain
    w_other_shape = moe.MoeWeights(dom, shared_expert=0, **make_experts(H, I, routed, seed=6, small=True))
    rejected(ws.run_quantized(w_other_shape, codes, scales, ids, routes, out))
    foreign = moe.MoeWeights(other, shared_expert=shared, **ex)
    assert ws.run_quantized(foreign, codes, scales, ids, routes, out) == capi.RK_NPU_ERR_DOMAIN
    assert np.array_equal(bits(out), bits(saved))
    # and the workspace still works
    assert ws.run_quantized(w, codes, scales, ids, routes, out) == 0 and np.array_equal(bits(out), bits(saved))
    for h in (foreign, w_other_shape, w):
        h.free()
    ws.free()


def test_constructors_validate(gpu):
    _, dom, _ = gpu
    lib = capi.load()
    ex = make_experts(64, 32, 2, seed=7, small=True)
    for field, value in (("gate_up_scales", 0.0), ("gate_up_scales", np.nan), ("down_scales", -1.0), ("down_scales", np.inf)):
        broken = {k: v.copy() for k, v in ex.items()}
        broken[field][1, 3] = value
        with pytest.raises(rk.W4A8Error):
            moe.MoeWeights(dom, shared_expert=0, **broken)
    for H, I, routed, shared in ((32, 32, 1, 0), (80, 32, 1, 0), (64, 16, 1, 0), (64, 544, 1, 0), (64, 48, 1, 0), (64, 32, 0, 0),
                                 (64, 32, 1, 2), (8224, 32, 1, 0)):
        cfg = capi.MoeWeightConfig(H, I, routed, shared)
        experts = (capi.MoeExpert * 4)()
        assert not lib.rk_npu_moe_w8_weights_create(dom.handle, C.byref(cfg), experts)
    good = moe.default_config(64, 32, 2, 0, 2, 8)
    for field, value in (("struct_size", 44), ("max_rows", 0), ("max_rows", 257), ("top_k", 0), ("top_k", 3), ("npu_cores", 0),
                         ("npu_cores", 4), ("cpu_threads", 5), ("native_input", 2), ("timeout_ms", 0), ("timeout_ms", 60001),
                         ("middle", 1), ("middle", 2)):
        c = capi.MoeConfig.from_buffer_copy(bytes(good))
        setattr(c, field, value)
        assert not lib.rk_npu_moe_w8_workspace_create(dom.handle, C.byref(c)), field
    c = capi.MoeConfig.from_buffer_copy(bytes(good))
    c.native_input = 1                                      # the original's other input layout: accepted, no effect here
    ws = moe.MoeWorkspace(dom, c)
    ws.free()


def test_empty_routes_and_single_expert(gpu, oracle):
    # tests/test_moe_w8.cpp:125-146: one expert, no shared one, every coefficient zero -> the output is cleared and
    # no device work is reported; scales are still validated
    _, dom, _ = gpu
    H, I = 64, 32
    ex = make_experts(H, I, 1, seed=8, small=True)
    w = moe.MoeWeights(dom, shared_expert=0, **ex)
    ws = moe.MoeWorkspace(dom, moe.default_config(H, I, 1, 0, 1, 256))
    for rows in (1, 128, 256):
        codes = np.ones((rows, H), np.int8)
        scales = np.full(rows, 0.03125, np.float32)
        ids = np.zeros((rows, 1), np.int32)
        routes = np.ones((rows, 1), np.float32)
        out = np.full((rows, H), 7.0, np.float32)
        rc_ref, ref = oracle.moe_run(ex, 0, 1, codes, scales, ids, routes, mode=1)
        assert ws.run_quantized(w, codes, scales, ids, routes, out) == 0 and np.array_equal(bits(out), bits(ref))
        routes[:] = 0
        t = capi.MoeTimings()
        assert ws.run_quantized(w, codes, scales, ids, routes, out, t) == 0
        assert not out.any() and t.gemm_tasks == t.gather_tasks == t.middle_tasks == 0 and t.sync_us == 0
        scales[0] = 0
        assert ws.run_quantized(w, codes, scales, ids, routes, out) == capi.RK_NPU_ERR_PARAM
    ws.free(); w.free()


def test_busy_workspace(gpu):
    import threading
    _, dom, _ = gpu
    H, I, routed, top, rows = 1536, 512, 8, 2, 256
    ex = make_experts(H, I, routed, seed=9)
    w = moe.MoeWeights(dom, shared_expert=0, **ex)
    ws = moe.MoeWorkspace(dom, moe.default_config(H, I, routed, 0, top, rows))
    rng = np.random.default_rng(0)
    codes = rng.integers(-127, 128, size=(rows, H), dtype=np.int8)
    scales = np.full(rows, 0.02, np.float32)
    ids, routes = make_routes(rows, routed, top, seed=1)
    outs = [np.zeros((rows, H), np.float32) for _ in range(4)]
    codes_seen = []

    def worker(o):
        for _ in range(20):
            codes_seen.append(ws.run_quantized(w, codes, scales, ids, routes, o))

    threads = [threading.Thread(target=worker, args=(o,)) for o in outs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert set(codes_seen) <= {0, capi.RK_NPU_ERR_BUSY} and 0 in codes_seen
    ws.free(); w.free()


@pytest.mark.parametrize("form", ["quant", "quant_full_k", "w4"])
@pytest.mark.parametrize("geometry", [(576, 64, 3, 1, 2), (128, 128, 4, 0, 2), (8128, 64, 3, 1, 2)], ids=lambda g: "x".join(map(str, g)))
def test_int4_expert_forms(gpu, oracle, form, geometry):
    # include/rk_npu_moe_w8.h:87-111: experts given as int8 arrays of int4 codes.  Accepted where the original certifies
    # the K tile its device would run (tests/test_moe_w8.cpp:68-69: a column of -8 overflows one INT16 partial over
    # K = 576 but fits 512 + 64); the numbers are those of the same codes run as int8 experts.
    _, dom, _ = gpu
    H, I, routed, shared, top = geometry
    E = routed + shared
    rng = np.random.default_rng(H + I)
    ex = dict(gate_up=rng.integers(-8, 8, size=(E, H, 2 * I), dtype=np.int8),
              gate_up_scales=rng.uniform(2e-3, 6e-3, size=(E, 2 * I)).astype(np.float32),
              down=rng.integers(-8, 8, size=(E, I, H), dtype=np.int8),
              down_scales=rng.uniform(1e-3, 3e-3, size=(E, H)).astype(np.float32))
    if H <= 2048:
        ex["gate_up"][1, 1:, 0] = -8            # needs the 512 + 64 split at K = 576
    if shared and form == "w4":
        ex["gate_up"][E - 1, 3, 5] = 100            # the shared expert of the mixed form is int8
    w = moe.MoeWeights(dom, shared_expert=shared, form=form, **ex)
    ws = moe.MoeWorkspace(dom, moe.default_config(H, I, routed, shared, top, 8), form=form)
    rows = 5
    codes = rng.integers(-128, 128, size=(rows, H), dtype=np.int8)
    scales = np.full(rows, 0.03125, np.float32)
    ids, routes = make_routes(rows, routed, top, seed=3)
    out = np.zeros((rows, H), np.float32)
    rc_ref, ref = oracle.moe_run(ex, shared, top, codes, scales, ids, routes, mode=1)
    assert rc_ref == 0 and ws.run_quantized(w, codes, scales, ids, routes, out) == 0
    assert np.array_equal(bits(out), bits(ref))
    # a workspace runs weights of its own form only (src/rk_npu_moe_w8.cpp:582)
    w8 = moe.MoeWeights(dom, shared_expert=shared, **{k: (np.clip(v, -8, 7) if v.dtype == np.int8 else v) for k, v in ex.items()})
    ws8 = moe.MoeWorkspace(dom, moe.default_config(H, I, routed, shared, top, 8))
    saved = out.copy()
    assert ws.run_quantized(w8, codes, scales, ids, routes, out) == capi.RK_NPU_ERR_PARAM
    assert ws8.run_quantized(w, codes, scales, ids, routes, out) == capi.RK_NPU_ERR_PARAM
    assert np.array_equal(bits(out), bits(saved))
    for h in (ws8, w8, ws, w):
        h.free()


def test_int4_expert_forms_validate(gpu, oracle):
    _, dom, _ = gpu
    lib = capi.load()
    H, I, E = 128, 64, 2
    rng = np.random.default_rng(2)

    def experts():
        return dict(gate_up=rng.integers(-8, 8, size=(E, H, 2 * I), dtype=np.int8), gate_up_scales=np.full((E, 2 * I), 1e-2, np.float32),
                    down=rng.integers(-8, 8, size=(E, I, H), dtype=np.int8), down_scales=np.full((E, H), 1e-2, np.float32))

    for form in ("quant", "quant_full_k", "w4"):
        for field, index, value in (("gate_up", (1, 7, 9), 8), ("gate_up", (0, 0, 0), -9), ("down", (1, 3, 3), 8), ("down", (0, 5, 1), -128)):
            ex = experts()
            ex[field][index] = value
            with pytest.raises(rk.W4A8Error):
                moe.MoeWeights(dom, shared_expert=0, form=form, **ex)      # a code outside [-8, 7]
        c = moe.default_config(H, I, E, 0, 2, 8)
        c.native_input = 1
        with pytest.raises(rk.W4A8Error):
            moe.MoeWorkspace(dom, c, form=form)                            # the int4 forms take normal input only
    # geometry: multiples of 64, hidden at most 8128
    for Hb, Ib in ((96, 64), (128, 96), (8192, 64)):
        cfg = capi.MoeWeightConfig(Hb, Ib, 1, 0)
        arr = (capi.MoeExpert * 1)()
        assert not lib.rk_npu_moe_quant_weights_create(dom.handle, C.byref(cfg), arr)
        assert not lib.rk_npu_moe_w4_weights_create(dom.handle, C.byref(cfg), arr)
        c = moe.default_config(Hb, Ib, 1, 0, 1, 8)
        assert not lib.rk_npu_moe_quant_workspace_create(dom.handle, C.byref(c))
    # certification follows the original's bound: a down matrix whose column sums overflow INT16 over K = 512 is refused,
    # the same column over K = 448 passes (oracle.bound restates src/rk_npu_i4_bounds.cpp)
    for Ib in (512, 448):
        ex = dict(gate_up=np.zeros((1, 64, 2 * Ib), np.int8), gate_up_scales=np.full((1, 2 * Ib), 1e-2, np.float32),
                  down=np.full((1, Ib, 64), -8, np.int8), down_scales=np.full((1, 64), 1e-2, np.float32))
        expect_ok = oracle.bound(ex["down"][0], requested=Ib)[0] == 0
        try:
            w = moe.MoeWeights(dom, shared_expert=0, form="quant", **ex)
            created = True
            w.free()
        except rk.W4A8Error:
            created = False
        assert created == expect_ok, Ib
