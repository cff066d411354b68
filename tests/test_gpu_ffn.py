"""Fused gate/up -> SwiGLU -> down through the C ABI.  Against the polynomial oracle the
whole chain is bit-exact; against the reference build's expf variant the staged bars of
the stated parity bars apply (middle <= 1e-6 relative, output <= 1e-3 relative)."""
import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from oracle.harness import make_activations, make_weights
from rknpu2_matmul_open_b200 import capi

pytestmark = pytest.mark.gpu


def build(dom, M, K, F, N, Bg, sg, Bd, sd, kt=480):
    wg, wd = rk.Weights(dom, Bg, sg, k_tile=kt), rk.Weights(dom, Bd, sd, k_tile=kt)
    g = rk.Workspace(dom, rk.default_config(M, 2 * F, K, k_tile=kt))
    d = rk.Workspace(dom, rk.default_config(M, N, F, k_tile=kt))
    return wg, wd, g, d


def free(*objs):
    for o in objs:
        o.free()


def test_reference_fixtures(gpu, oracle, golden_ffn):
    _, dom, _ = gpu
    g = golden_ffn
    for i in range(int(g["count"])):
        t = f"f{i}"
        M, K, F, N = (int(x) for x in g[f"{t}_shape"])
        wg, wd, gu, dn = build(dom, M, K, F, N, g[f"{t}_Bg"], g[f"{t}_sg"], g[f"{t}_Bd"], g[f"{t}_sd"])
        middle, C = np.zeros((M, F), np.float32), np.zeros((M, N), np.float32)
        assert rk.run_ffn_f32(gu, wg, dn, wd, g[f"{t}_A"], middle, C) == 0
        ref_mid, ref_c = g[f"{t}_middle"], g[f"{t}_C"]
        assert np.all(np.abs(middle - ref_mid) <= 1e-6 * np.abs(ref_mid) + 1e-30)
        assert np.all(np.abs(C - ref_c) <= 1e-3 * np.abs(ref_c) + 1e-6)
        poly = oracle.ffn(g[f"{t}_A"], g[f"{t}_Bg"], g[f"{t}_sg"], g[f"{t}_Bd"], g[f"{t}_sd"], mode=1)
        assert np.array_equal(bits(middle), bits(poly["middle"])) and np.array_equal(bits(C), bits(poly["C"]))
        free(gu, dn, wg, wd)


# M x F x K grid of the reference's SwiGLU/FFN tests (F 96 and 992 are 32 mod 64)
CASES = [(1, 479, 96, 192), (9, 959, 128, 192), (65, 1057, 992, 192), (2, 479, 128, 64), (4, 959, 128, 257),
         (8, 1057, 9728, 128), (64, 479, 128, 65), (65, 959, 96, 193), (128, 1057, 128, 129), (33, 4096, 1024, 512)]


@pytest.mark.parametrize("case", CASES, ids=lambda s: "x".join(map(str, s)))
def test_ffn_equals_staged_operators_bit_for_bit(gpu, oracle, case):
    _, dom, _ = gpu
    M, K, F, N = case
    Bg, sg = make_weights(K, 2 * F, seed=F)
    Bd, sd = make_weights(F, N, seed=N)
    wg, wd, gu, dn = build(dom, M, K, F, N, Bg, sg, Bd, sd)
    for pattern in range(3):
        A = make_activations(M, K, seed=pattern, dtype="f32")
        if pattern == 1:
            A[:] = 0                                       # zero input: zero middle, scale 1, zero output
        if pattern == 2:
            A = -np.abs(A)
        middle, C = np.zeros((M, F), np.float32), np.zeros((M, N), np.float32)
        t = capi.W4A8FfnTimings()
        assert rk.run_ffn_f32(gu, wg, dn, wd, A, middle, C, t) == 0
        assert t.down.activation_scan_us == 0              # down never rescans: scales come from the epilogue
        ref = oracle.ffn(A, Bg, sg, Bd, sd, mode=1)
        assert np.array_equal(ref["acc_gate_up"], _acc(gu, wg, A))
        assert np.array_equal(bits(middle), bits(ref["middle"]))
        assert np.array_equal(bits(C), bits(ref["C"]))
        # fused == separate SwiGLU call followed by an ordinary linear on middle
        only = np.zeros((M, F), np.float32)
        assert gu.run_swiglu_f32(wg, A, only) == 0 and np.array_equal(bits(only), bits(middle))
        C2 = np.zeros((M, N), np.float32)
        assert dn.run_f32(wd, middle, C2) == 0 and np.array_equal(bits(C2), bits(C))
        rc, s, q = dn.last_quant()
        assert np.array_equal(bits(s), bits(ref["scales_down_in"]))       # reused scale == rescanned scale
        if pattern == 1:
            assert not middle.any() and not C.any()
    free(gu, dn, wg, wd)


def _acc(ws, w, A):
    acc = np.zeros((A.shape[0], ws.cfg.N), np.int32)
    assert ws.run_acc_i32(w, A, acc) == 0
    return acc


def test_nonfinite_middle_is_rejected_before_down(gpu, oracle):
    # w_scale = FLT_MAX drives middle to inf: PARAM after gate/up, down does no work
    _, dom, _ = gpu
    M, K, F, N = 3, 959, 128, 256
    Bg = np.ones((K, 2 * F), np.int8)
    sg = np.full(2 * F, np.finfo(np.float32).max, np.float32)
    Bd, sd = make_weights(F, N, seed=1)
    wg, wd, gu, dn = build(dom, M, K, F, N, Bg, sg, Bd, sd)
    A = np.abs(make_activations(M, K, seed=1, dtype="f32")) + 1
    middle, C = np.zeros((M, F), np.float32), np.full((M, N), 7.0, np.float32)
    t = capi.W4A8FfnTimings()
    assert rk.run_ffn_f32(gu, wg, dn, wd, A, middle, C, t) == capi.RK_NPU_ERR_PARAM
    assert t.down.submit_us == 0
    assert oracle.ffn(A, Bg, sg, Bd, sd, mode=1)["rc"] == -3
    # NaN input is refused too, and both workspaces stay usable
    A2 = make_activations(M, K, seed=2, dtype="f32")
    A2[1, 1] = np.nan
    assert rk.run_ffn_f32(gu, wg, dn, wd, A2, middle, C) == capi.RK_NPU_ERR_PARAM
    free(gu, dn, wg, wd)
    Bg, sg = make_weights(K, 2 * F, seed=3)
    wg, wd, gu, dn = build(dom, M, K, F, N, Bg, sg, Bd, sd)
    A3 = make_activations(M, K, seed=3, dtype="f32")
    assert rk.run_ffn_f32(gu, wg, dn, wd, A3, middle, C) == 0
    assert np.array_equal(bits(C), bits(oracle.ffn(A3, Bg, sg, Bd, sd, mode=1)["C"]))
    free(gu, dn, wg, wd)


def test_ffn_argument_errors(gpu):
    ctx, dom, other = gpu
    lib = capi.load()
    M, K, F, N = 4, 256, 64, 96
    Bg, sg = make_weights(K, 2 * F, seed=1)
    Bd, sd = make_weights(F, N, seed=2)
    wg, wd, gu, dn = build(dom, M, K, F, N, Bg, sg, Bd, sd)
    A = make_activations(M, K, seed=1, dtype="f32")
    middle, C = np.zeros((M, F), np.float32), np.zeros((M, N), np.float32)
    t = capi.W4A8FfnTimings()
    t.total_us = 5
    assert lib.rk_npu_w4a8_run_ffn_f32(None, wg.handle, dn.handle, wd.handle, A.ctypes.data, middle.ctypes.data,
                                       C.ctypes.data, t) == -3 and t.total_us == 0          # timings are zeroed
    assert rk.run_ffn_f32(gu, wg, gu, wg, A, middle, C) == -3                                # same workspace twice
    assert rk.run_ffn_f32(gu, wg, dn, wd, A, middle, middle) == -3                           # aliasing
    wrong = rk.Workspace(dom, rk.default_config(M + 1, N, F))
    assert rk.run_ffn_f32(gu, wg, wrong, wd, A, middle, C) == -3                             # M mismatch
    wrong.free()
    wrong = rk.Workspace(dom, rk.default_config(M, N, F + 32))
    wd2 = rk.Weights(dom, *make_weights(F + 32, N, seed=3))
    assert rk.run_ffn_f32(gu, wg, wrong, wd2, A, middle, C) == -3                            # F mismatch
    free(wrong, wd2)
    dn_other = rk.Workspace(other, rk.default_config(M, N, F))
    wd_other = rk.Weights(other, Bd, sd)
    assert rk.run_ffn_f32(gu, wg, dn_other, wd_other, A, middle, C) == capi.RK_NPU_ERR_DOMAIN
    free(dn_other, wd_other)
    # SwiGLU needs N % 64 == 0
    odd = rk.Workspace(dom, rk.default_config(M, 96, K))
    w_odd = rk.Weights(dom, *make_weights(K, 96, seed=4))
    assert odd.run_swiglu_f32(w_odd, A, np.zeros((M, 48), np.float32)) == -3
    free(odd, w_odd, gu, dn, wg, wd)


def test_full_size_ffn_decode(gpu, oracle):
    # benchmark configuration 3 at M = 1: 4096 -> 2 x 14336 -> 4096, whole chain bit-exact vs the oracle
    _, dom, _ = gpu
    M, K, F, N = 1, 4096, 14336, 4096
    Bg, sg = make_weights(K, 2 * F, seed=31)
    Bd, sd = make_weights(F, N, seed=32)
    wg, wd, gu, dn = build(dom, M, K, F, N, Bg, sg, Bd, sd)
    A = make_activations(M, K, seed=31, dtype="f32")
    middle, C = np.zeros((M, F), np.float32), np.zeros((M, N), np.float32)
    assert rk.run_ffn_f32(gu, wg, dn, wd, A, middle, C) == 0
    ref = oracle.ffn(A, Bg, sg, Bd, sd, mode=1)
    assert np.array_equal(bits(middle), bits(ref["middle"])) and np.array_equal(bits(C), bits(ref["C"]))
    free(gu, dn, wg, wd)


# the FFN through every small-batch schedule (SwiGLU epilogue + row-maximum reuse in each GEMM kernel)
@pytest.mark.parametrize("variant", [1, 3, 4])
@pytest.mark.parametrize("case", [(1, 1057, 992, 192), (8, 2304, 1600, 300), (20, 479, 96, 65), (32, 4096, 1024, 512),
                                  (70, 1057, 992, 192), (128, 4096, 1024, 512)],
                         ids=lambda s: "x".join(map(str, s)))
def test_ffn_small_batch_schedules_agree(gpu, oracle, monkeypatch, variant, case):
    _, dom, _ = gpu
    monkeypatch.setenv("RK_NPU_B200_VARIANT", str(variant))
    M, K, F, N = case
    Bg, sg = make_weights(K, 2 * F, seed=F + 1)
    Bd, sd = make_weights(F, N, seed=N + 1)
    wg, wd, gu, dn = build(dom, M, K, F, N, Bg, sg, Bd, sd)
    for rep in range(2):
        A = make_activations(M, K, seed=rep, dtype="f32")
        middle, C = np.zeros((M, F), np.float32), np.zeros((M, N), np.float32)
        assert rk.run_ffn_f32(gu, wg, dn, wd, A, middle, C, None) == 0
        ref = oracle.ffn(A, Bg, sg, Bd, sd, mode=1)
        assert np.array_equal(bits(middle), bits(ref["middle"]))
        assert np.array_equal(bits(C), bits(ref["C"]))
    free(gu, dn, wg, wd)


# The column-sharded FFN's code exchange, with the "ranks" run one after another on this GPU: per-slice SwiGLU with
# collected row maxima, maxima combined, slices quantised with the combined scale, codes stacked as an all-gather
# would leave them, down projection per column shard on the stacked codes.  Must equal the unsharded chain.
@pytest.mark.parametrize("case", [(1, 479, 128, 192, 2), (8, 1057, 1024, 256, 4), (33, 959, 512, 320, 2),
                                  (160, 1057, 2048, 512, 4), (5, 4096, 4096, 4096, 8)],
                         ids=lambda s: "x".join(map(str, s)))
def test_sharded_ffn_code_exchange_is_bit_exact(gpu, oracle, case):
    import torch
    from rknpu2_matmul_open_b200.sharding import shard_ffn_weights, shard_weights
    _, dom, _ = gpu
    M, K, F, N, g = case
    Bg, sg = make_weights(K, 2 * F, seed=F + 2)
    Bd, sd = make_weights(F, N, seed=N + 2)
    A = make_activations(M, K, seed=g, dtype="f32")
    ref = oracle.ffn(A, Bg, sg, Bd, sd, mode=1)
    dev = torch.device("cuda:0")
    dA = torch.from_numpy(A).to(dev)
    pc = F // g
    maxima = [torch.zeros(M, dtype=torch.int32, device=dev) for _ in range(g)]
    middles, handles = [], []
    for r in range(g):
        Bs, ss, (f0, f1) = shard_ffn_weights(Bg, sg, g, r)
        assert f1 - f0 == pc
        w = rk.Weights(dom, Bs, ss)
        ws = rk.Workspace(dom, rk.default_config(M, 2 * pc, K))
        mid = torch.zeros((M, pc), dtype=torch.float32, device=dev)
        assert ws.enqueue_swiglu_collect_f32(w, dA, mid, maxima[r]) == 0
        middles.append(mid)
        handles.append((w, ws))
    torch.cuda.synchronize()
    middle = torch.cat(middles, dim=1).cpu().numpy()
    assert np.array_equal(bits(middle), bits(ref["middle"]))
    combined = torch.stack(maxima).max(dim=0).values.contiguous()          # what the integer all-reduce(max) gives
    assert np.array_equal(combined.cpu().numpy().view(np.uint32), np.abs(ref["middle"]).max(axis=1).view(np.uint32))
    codes = torch.zeros((g, M, pc), dtype=torch.int8, device=dev)
    for r, (w, ws) in enumerate(handles):
        assert ws.enqueue_quantize_slice(middles[r], combined, codes[r]) == 0
    torch.cuda.synchronize()
    out = np.zeros((M, N), np.float32)
    for r in range(g):
        Bs, ss, (n0, n1) = shard_weights(Bd, sd, g, r)
        if n1 == n0:
            continue
        w = rk.Weights(dom, Bs, ss)
        ws = rk.Workspace(dom, rk.default_config(M, n1 - n0, F))
        dC = torch.zeros((M, n1 - n0), dtype=torch.float32, device=dev)
        mx = combined.clone()
        assert ws.enqueue_codes_f32(w, codes, g, mx, dC) == 0
        torch.cuda.synchronize()
        assert ws.finish() == 0
        assert int(mx.abs().sum()) == 0                                      # consumed and cleared
        out[:, n0:n1] = dC.cpu().numpy()
        free(ws, w)
    assert np.array_equal(bits(out), bits(ref["C"]))
    for w, ws in handles:
        free(ws, w)


def test_codes_entry_plain_matrix_and_errors(gpu, oracle):
    """parts = 1 takes a plain [M, K] code matrix (any K); a non-finite maximum is reported after the run."""
    import torch
    _, dom, _ = gpu
    M, K, N = 7, 1001, 130
    B, sw = make_weights(K, N, seed=9)
    X = make_activations(M, K, seed=9, dtype="f32")
    ref_rc, ref, _, _ = oracle.linear(X, B, sw)
    assert ref_rc == 0
    dev = torch.device("cuda:0")
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    # the same linear through the ordinary entry gives the codes and the reference output
    dC0 = torch.zeros((M, N), dtype=torch.float32, device=dev)
    assert ws.enqueue_f32(w, torch.from_numpy(X).to(dev), dC0) == 0
    torch.cuda.synchronize()
    acc = np.zeros((M, N), np.int32)
    assert ws.run_acc_i32(w, X, acc) == 0
    rc, scales, q = ws.last_quant()
    assert rc == 0
    maxima = torch.from_numpy(np.abs(X).max(axis=1).view(np.int32).copy()).to(dev)
    dC = torch.zeros((M, N), dtype=torch.float32, device=dev)
    assert ws.enqueue_codes_f32(w, torch.from_numpy(q).to(dev), 1, maxima, dC) == 0
    torch.cuda.synchronize()
    assert ws.finish() == 0
    assert np.array_equal(bits(dC.cpu().numpy()), bits(dC0.cpu().numpy()))
    assert np.array_equal(bits(dC.cpu().numpy()), bits(ref))
    # argument errors: parts must divide K into multiples of 16
    assert ws.enqueue_codes_f32(w, torch.from_numpy(q).to(dev), 7, maxima, dC) == capi.RK_NPU_ERR_PARAM
    assert ws.enqueue_codes_f32(w, torch.from_numpy(q).to(dev), 0, maxima, dC) == capi.RK_NPU_ERR_PARAM
    # an infinite row maximum: the GEMM does not write, finish reports PARAM, the workspace stays usable
    bad = torch.from_numpy(np.full(M, 0x7f800000, np.int32)).to(dev)
    dC.fill_(7.0)
    assert ws.enqueue_codes_f32(w, torch.from_numpy(q).to(dev), 1, bad, dC) == 0
    torch.cuda.synchronize()
    assert ws.finish() == capi.RK_NPU_ERR_PARAM
    assert float(dC.min()) == 7.0
    assert ws.enqueue_f32(w, torch.from_numpy(X).to(dev), dC) == 0
    torch.cuda.synchronize()
    assert ws.finish() == 0
    assert np.array_equal(bits(dC.cpu().numpy()), bits(dC0.cpu().numpy()))
    free(ws, w)


@pytest.mark.parametrize("case", [(1, 1057, 992, 192), (8, 2304, 1600, 300), (20, 479, 192, 257)],
                         ids=lambda s: "x".join(map(str, s)))
def test_ffn_single_kernel_two_tiles_per_cta(gpu, oracle, monkeypatch, case):
    """SwiGLU epilogue, collected row maxima and their reuse with two column tiles per CTA."""
    _, dom, _ = gpu
    monkeypatch.setenv("RK_NPU_B200_VARIANT", "3")
    monkeypatch.setenv("RK_NPU_B200_TILES_PER_CTA", "2")
    M, K, F, N = case
    Bg, sg = make_weights(K, 2 * F, seed=F + 3)
    Bd, sd = make_weights(F, N, seed=N + 3)
    wg, wd, gu, dn = build(dom, M, K, F, N, Bg, sg, Bd, sd)
    for rep in range(2):
        A = make_activations(M, K, seed=rep, dtype="f32")
        middle, C = np.zeros((M, F), np.float32), np.zeros((M, N), np.float32)
        assert rk.run_ffn_f32(gu, wg, dn, wd, A, middle, C, None) == 0
        ref = oracle.ffn(A, Bg, sg, Bd, sd, mode=1)
        assert np.array_equal(bits(middle), bits(ref["middle"]))
        assert np.array_equal(bits(C), bits(ref["C"]))
    free(gu, dn, wg, wd)
