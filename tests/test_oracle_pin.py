"""The oracle (oracle/w4a8_oracle.c) against what pins it: fixtures generated from the
reference's compiled CPU stages (tests/golden), the known answers the reference's own
tests assert, and -- where it was built -- the reference code itself on fresh inputs."""
import numpy as np
import pytest

from conftest import bits
from oracle.harness import make_activations, make_weights, sample_columns

FLT_MIN = np.float32(1.17549435e-38)


def test_half_tables_match_reference(oracle, golden_half):
    halves = np.arange(65536, dtype=np.uint16)
    assert np.array_equal(bits(oracle.half_to_float(halves)), golden_half["h2f"])
    f_in = golden_half["f_in"].view(np.float32)
    assert np.array_equal(oracle.float_to_half(f_in), golden_half["f2h"])


def test_half_round_trip_is_exhaustive(oracle):
    # every finite binary16 pattern survives half -> float -> half (tests/test_w4a8_cpu.cpp:122-128)
    halves = np.arange(65536, dtype=np.uint16)
    f = oracle.half_to_float(halves)
    keep = ~np.isnan(f)
    assert np.array_equal(oracle.float_to_half(f)[keep], halves[keep])
    assert np.array_equal(bits(f), bits(halves.view(np.float16).astype(np.float32)))


def test_linear_matches_reference_fixtures(oracle, golden_linear):
    g = golden_linear
    for i in range(int(g["count"])):
        t = f"c{i}"
        for A, out, acc, s, q in ((g[f"{t}_A32"], g[f"{t}_out32"], g[f"{t}_acc32"], g[f"{t}_s32"], g[f"{t}_q32"]),
                                  (g[f"{t}_A16"], g[f"{t}_out16"], g[f"{t}_acc16"], g[f"{t}_s16"], g[f"{t}_q16"])):
            rc, o_out, o_acc, o_s = oracle.linear(A, g[f"{t}_B"], g[f"{t}_sw"])
            assert rc == 0
            assert np.array_equal(o_acc, acc), f"case {i}: int32 accumulators"
            assert np.array_equal(bits(o_out), bits(out)), f"case {i}: output"
            assert np.array_equal(bits(o_s), bits(s)), f"case {i}: scales"
            _, _, inv = oracle.scales(A)
            assert np.array_equal(oracle.quantize(A, inv), q), f"case {i}: codes"


def test_ffn_expf_matches_reference_fixtures(oracle, golden_ffn):
    g = golden_ffn
    for i in range(int(g["count"])):
        t = f"f{i}"
        r = oracle.ffn(g[f"{t}_A"], g[f"{t}_Bg"], g[f"{t}_sg"], g[f"{t}_Bd"], g[f"{t}_sd"], mode=0)
        assert r["rc"] == 0
        assert np.array_equal(bits(r["middle"]), bits(g[f"{t}_middle"]))
        assert np.array_equal(bits(r["scales_down_in"]), bits(g[f"{t}_scales_down"]))
        assert np.array_equal(bits(r["C"]), bits(g[f"{t}_C"]))


def test_polynomial_silu_tracks_expf(oracle, golden_ffn):
    # the reference asserts <= 7e-7 relative between its polynomial and expf
    # (tests/test_w4a8_swiglu.cpp:44-71), including the saturated ends
    xs = np.concatenate([np.linspace(-90, 90, 20001), [-100, 100, -80, 80, -80.00001, 0.0, -0.0, 3.4e38, -3.4e38]])
    for x in xs.astype(np.float32):
        p, e = oracle.lib.orc_silu_poly(float(x)), oracle.lib.orc_silu_expf(float(x))
        if x < -80:
            assert p == 0.0 and np.signbit(np.float32(p))
        else:
            assert abs(p - e) <= 7e-7 * abs(e) + 1e-37, x
    g = golden_ffn
    for i in range(int(g["count"])):
        t = f"f{i}"
        r = oracle.ffn(g[f"{t}_A"], g[f"{t}_Bg"], g[f"{t}_sg"], g[f"{t}_Bd"], g[f"{t}_sd"], mode=1)
        ref_mid = g[f"{t}_middle"]
        assert np.all(np.abs(r["middle"] - ref_mid) <= 1e-6 * np.abs(ref_mid) + 1e-30)
        ref_c = g[f"{t}_C"]
        assert np.all(np.abs(r["C"] - ref_c) <= 1e-3 * np.abs(ref_c) + 1e-6)


def test_quantizer_edge_rows(oracle):
    # tests/test_w4a8_cpu.cpp:20-89: zero row, scaled ramps, full-row maximum in the last
    # element, exact ties, non-finite rejection, denormal -> FLT_MIN
    M, K = 5, 533
    a = np.zeros((M, K), np.float32)
    for m in range(1, M):
        a[m] = np.ldexp((np.arange(K) % 255 - 127).astype(np.float32), m - 3)
        a[m, K - 1] = np.ldexp(np.float32(254), m - 3)
    a[1] = (np.arange(K) % 255 - 127).astype(np.float32)
    a[1, 1:5] = [.5, -.5, 1.5, -1.5]
    a[1, K - 2] = -.5
    for A in (a, oracle.float_to_half(a)):
        rc, s, inv = oracle.scales(A)
        assert rc == 0 and s[0] == 1
        q = oracle.quantize(A, inv)
        f = A if A.dtype == np.float32 else oracle.half_to_float(A)
        mx = np.abs(f).max(axis=1)
        exp_s = np.where(mx == 0, np.float32(1), np.maximum(mx / np.float32(127), FLT_MIN)).astype(np.float32)
        assert np.array_equal(bits(s), bits(exp_s))
        prod = (f * (np.float32(1) / exp_s)[:, None]).astype(np.float32)
        exp_q = np.clip(np.sign(prod) * np.floor(np.abs(prod) + np.float32(0.5)), -127, 127).astype(np.int8)
        assert np.array_equal(q, exp_q)
    assert list(oracle.quantize(a, np.ones(M, np.float32))[1, 1:5]) == [1, -1, 2, -2]   # ties away from zero
    bad = a.copy()
    bad[0, 0] = np.inf
    assert oracle.scales(bad)[0] == -3
    bad[0, 0] = np.nan
    assert oracle.scales(bad)[0] == -3
    h = oracle.float_to_half(a)
    h[0, 0] = 0x7c00
    assert oracle.scales(h)[0] == -3
    rc, s, inv = oracle.scales(np.array([[1e-45]], np.float32))
    assert rc == 0 and s[0] == FLT_MIN and np.isfinite(inv[0])


def test_dequant_expression(oracle):
    # tests/test_w4a8_cpu.cpp:133-142: (float(acc) * a_scale) * w_scale, then one fp16 rounding
    acc = np.array([[1 << 25, -(1 << 25) - 3, 7, 0, 123456789]], np.int32)
    a_s = np.array([0.37], np.float32)
    w_s = np.array([0.011, 3.0, 1e-3, 5.0, 2.5e-4], np.float32)
    exp = ((acc.astype(np.float32) * a_s[:, None]).astype(np.float32) * w_s).astype(np.float32)
    assert np.array_equal(bits(oracle.dequant(acc, a_s, w_s, False)), bits(exp))
    assert np.array_equal(oracle.dequant(acc, a_s, w_s, True), oracle.float_to_half(exp))


def test_finish_scales_boundaries(oracle):
    # tests/test_w4a8_ffn.cpp:18-36
    as_bits = lambda x: np.array([x], np.float32).view(np.uint32)[0]
    rc, s, inv = oracle.finish_scales(np.array([0, as_bits(1e-45), as_bits(FLT_MIN), as_bits(2.0)], np.uint32))
    assert rc == 0 and s[0] == 1 and s[1] == FLT_MIN and s[2] == FLT_MIN
    assert s[3] == np.float32(2.0) / np.float32(127) and inv[3] == np.float32(1) / s[3]
    assert oracle.finish_scales(np.array([0x7f800000], np.uint32))[0] == -3
    assert oracle.finish_scales(np.array([0x7fc00000], np.uint32))[0] == -3


def test_bound_known_answers(oracle):
    # tests/test_i4_bounds.cpp:14-42
    w = np.full((2048, 1), -8, np.int8)
    rc, kt, pos, neg, mask = oracle.bound(w)
    assert rc == 0 and kt == 480
    assert oracle.bound(w, 512)[0] == -3
    assert oracle.bound(w, 2048, 512)[0] == -3
    rc, kt, pos, neg, _ = oracle.bound(w[:511], 512)
    assert rc == 0 and pos == 32704
    w[:] = 4
    rc, kt, pos, neg, _ = oracle.bound(w)
    assert rc == 0 and kt == 1024 and neg == 32768
    rc, kt, pos, neg, _ = oracle.bound(w, 2048, 512)
    assert rc == 0 and kt == 512 and neg == 16384
    w[:] = 0
    assert oracle.bound(w, 2048, 512)[1] == 2048
    w[624:1424] = -8
    assert oracle.bound(w, 768)[0] == -3
    assert oracle.bound(w, 1024)[0] == 0
    assert oracle.bound(w)[1] == 1120       # safety is not monotonic in the tile size
    w = np.zeros((2048, 129), np.int8)
    w[:, 128] = -8
    assert oracle.bound(w)[1] == 480        # the last column of the second slab decides
    w[-1, -1] = 8
    assert oracle.bound(w)[0] == -3
    assert oracle.bound(w, 2048, 512)[0] == -3


def test_weight_rules(oracle):
    B, sw = make_weights(64, 48, seed=9)
    rc, corr = oracle.weight_check(B, sw)
    assert rc == 0 and np.array_equal(corr, 8 * B.astype(np.int32).sum(axis=0))
    for bad in (0.0, np.inf, -1.0, np.nan):
        s2 = sw.copy()
        s2[3] = bad
        assert oracle.weight_check(B, s2)[0] == -3
    B2 = B.copy()
    B2[0, 0] = 8
    assert oracle.weight_check(B2, sw)[0] == -3


# ------------------------------------------------------------------ live checks against the reference build
def test_against_reference_build_linear(oracle, reference):
    for (M, K, N, kt) in [(16, 2048, 2048, 480), (16, 2048, 2048, 2048), (1, 4096, 4096, 480), (65, 1921, 1025, 480)]:
        B, sw = make_weights(K, N, seed=M)
        for dtype in ("f16", "f32"):
            A = make_activations(M, K, seed=M, dtype=dtype)
            r = reference.linear(A, B, sw, k_tile=kt, threads=4)
            rc, out, acc, s = oracle.linear(A, B, sw)
            assert r["rc"] == 0 and rc == 0 and r["saturated"] == 0
            assert np.array_equal(acc, r["acc"]) and np.array_equal(bits(out), bits(r["out"]))
            assert np.array_equal(bits(s), bits(r["scales"]))


def test_against_reference_build_sampled_large(oracle, reference):
    # decode shape at full size: 17 evenly spaced columns x all rows, as the reference samples
    M, K, N = 8, 4096, 11008
    B, sw = make_weights(K, N, seed=1)
    A = make_activations(M, K, seed=1, dtype="f16")
    r = reference.linear(A, B, sw, k_tile=480, threads=4, want_acc=True)
    cols = sample_columns(N)
    _, _, inv = oracle.scales(A)
    acc = oracle.gemm_i32_columns(oracle.quantize(A, inv), B, cols)
    assert np.array_equal(acc, r["acc"][:, cols])


def test_against_reference_build_ffn(oracle, reference):
    for (M, K, F, N) in [(8, 1024, 2048, 1024), (33, 1057, 992, 512), (1, 479, 96, 192)]:
        Bg, sg = make_weights(K, 2 * F, seed=11)
        Bd, sd = make_weights(F, N, seed=12)
        A = make_activations(M, K, seed=11, dtype="f32")
        r = reference.ffn(A, Bg, sg, Bd, sd, threads=3)
        o = oracle.ffn(A, Bg, sg, Bd, sd, mode=0)
        assert r["rc"] == 0 and o["rc"] == 0
        assert np.array_equal(bits(o["middle"]), bits(r["middle"]))
        assert np.array_equal(bits(o["C"]), bits(r["C"]))
        only = reference.ffn(A, Bg, sg, None, None, swiglu_only=True)
        assert np.array_equal(bits(only["middle"]), bits(r["middle"]))


def test_against_reference_build_bounds_and_fingerprint(oracle, reference):
    rng = np.random.Generator(np.random.PCG64(5))
    for (K, N) in [(2048, 129), (1500, 300), (4096, 64)]:
        B = rng.integers(-8, 8, size=(K, N), dtype=np.int8)
        sw = rng.random(N, dtype=np.float32) + np.float32(0.01)
        assert oracle.bound(B) == reference.bound(B)
        assert oracle.bound(B, 992, 480) == reference.bound(B, 992, 480)
        assert oracle.fingerprint(B, sw) == reference.fingerprint(B, sw)
    B, sw = make_weights(4096, 256, seed=2)
    assert oracle.bound(B) == reference.bound(B)
