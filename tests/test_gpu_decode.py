"""The decode kernel (up to eight tokens; a CTA owns whole output channels over all of K, the CTAs of a
cluster share the quantisation and exchange int8 codes) through the C ABI against the oracle.

Covered: every token count 1..8 with every cluster size (the split of the quantisation work changes with
both), K tails and K beyond one ring pass, channel tails, more weight groups than CTAs (several items per
CTA, the ring wraps between items), both input types, the exact int32 sums, the fused FFN (SwiGLU pairs,
collected row maxima feeding the down projection without a rescan), rejected inputs, and one workspace
reused many times.  Everything is compared bit for bit.
"""
import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from oracle.harness import make_activations, make_weights
from rknpu2_matmul_open_b200 import capi

pytestmark = pytest.mark.gpu


def linear_case(dom, oracle, M, K, N, dtype, cluster, seed):
    B, sw = make_weights(K, N, seed=seed)
    A = make_activations(M, K, seed=seed + 1, dtype=dtype)
    if M > 2:
        A[M - 2, :] = 0
    half = dtype == "f16"
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    assert ws.set_schedule(5, cluster) == 0, "the workspace does not run the decode kernel"
    out = np.full((M, N), 0x5555 if half else -12345.0, np.uint16 if half else np.float32)
    acc = np.zeros((M, N), np.int32)
    assert (ws.run_f16 if half else ws.run_f32)(w, A, out) == 0
    assert ws.run_acc_i32(w, A, acc) == 0
    rc, s, q = ws.last_quant()
    ws.free()
    w.free()
    rc, ref, ref_acc, ref_s = oracle.linear(A, B, sw)
    assert rc == 0
    _, _, inv = oracle.scales(A)
    assert np.array_equal(bits(s), bits(ref_s)), "token scales"
    assert np.array_equal(q, oracle.quantize(A, inv)), "int8 codes"
    assert np.array_equal(acc, ref_acc), "int32 sums"
    assert np.array_equal(bits(out), bits(ref)), "output"


@pytest.mark.parametrize("cluster", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 6, 7, 8])
def test_every_token_count_and_cluster_size(gpu, oracle, M, cluster):
    _, dom, _ = gpu
    for (K, N, dtype) in [(1057, 193, "f16"), (2304, 1000, "f32")]:
        linear_case(dom, oracle, M, K, N, dtype, cluster, seed=10 * M + cluster)


@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 33, 65), (8, 4096, 4096), (1, 4096, 4096), (8, 11008, 4096), (8, 4096, 11008),
                                   (5, 16384, 160), (2, 20003, 65), (8, 1024, 14241), (4, 1441, 9999), (7, 513, 4737)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_shapes(gpu, oracle, shape, dtype):
    _, dom, _ = gpu
    M, K, N = shape
    linear_case(dom, oracle, M, K, N, dtype, 0, seed=K + N)


@pytest.mark.parametrize("cluster", [0, 1, 8])
@pytest.mark.parametrize("case", [(1, 479, 96, 192), (2, 959, 128, 257), (8, 1057, 9728, 128), (7, 1057, 992, 192), (5, 4096, 4768, 320)],
                         ids=lambda s: "x".join(map(str, s)))
def test_ffn(gpu, oracle, case, cluster):
    _, dom, _ = gpu
    M, K, F, N = case
    Bg, sg = make_weights(K, 2 * F, seed=F)
    Bd, sd = make_weights(F, N, seed=N)
    wg, wd = rk.Weights(dom, Bg, sg), rk.Weights(dom, Bd, sd)
    gu = rk.Workspace(dom, rk.default_config(M, 2 * F, K))
    dn = rk.Workspace(dom, rk.default_config(M, N, F))
    assert gu.set_schedule(5, cluster) == 0 and dn.set_schedule(5, cluster) == 0
    for pattern in range(3):
        A = make_activations(M, K, seed=pattern, dtype="f32")
        if pattern == 1:
            A[:] = 0
        if pattern == 2:
            A = -np.abs(A)
        middle, C = np.zeros((M, F), np.float32), np.zeros((M, N), np.float32)
        t = capi.W4A8FfnTimings()
        assert rk.run_ffn_f32(gu, wg, dn, wd, A, middle, C, t) == 0
        ref = oracle.ffn(A, Bg, sg, Bd, sd, mode=1)
        assert np.array_equal(bits(middle), bits(ref["middle"]))
        assert np.array_equal(bits(C), bits(ref["C"]))
        rc, s, q = dn.last_quant()
        assert np.array_equal(bits(s), bits(ref["scales_down_in"]))
        only = np.zeros((M, F), np.float32)
        assert gu.run_swiglu_f32(wg, A, only) == 0 and np.array_equal(bits(only), bits(middle))
    for x in (gu, dn, wg, wd):
        x.free()


def test_rejected_inputs_and_reuse(gpu, oracle):
    _, dom, _ = gpu
    M, K, N = 6, 3000, 1500
    B, sw = make_weights(K, N, seed=9)
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    assert ws.set_schedule(5, 0) == 0
    out = np.zeros((M, N), np.float32)
    for rep in range(5):
        A = make_activations(M, K, seed=rep, dtype="f32")
        assert ws.run_f32(w, A, out) == 0
        assert np.array_equal(bits(out), bits(oracle.linear(A, B, sw)[1])), rep
    for (row, col, value) in [(0, 0, np.nan), (M - 1, K - 1, np.inf), (3, 1717, -np.inf)]:
        bad = make_activations(M, K, seed=1, dtype="f32")
        bad[row, col] = value
        t = capi.W4A8Timings()
        assert ws.run_f32(w, bad, out, t) == capi.RK_NPU_ERR_PARAM
        assert t.total_us < 100e3                            # refused without waiting for a time limit to run out
        bad16 = oracle.float_to_half(np.where(np.isfinite(bad), bad, 0).astype(np.float32))
        bad16[row, col] = 0x7C00 if value == np.inf else 0xFC00 if value == -np.inf else 0x7E01
        out16 = np.zeros((M, N), np.uint16)
        assert ws.run_f16(w, bad16, out16) == capi.RK_NPU_ERR_PARAM
    A = make_activations(M, K, seed=77, dtype="f32")
    assert ws.run_f32(w, A, out) == 0
    assert np.array_equal(bits(out), bits(oracle.linear(A, B, sw)[1]))
    ws.free()
    w.free()


@pytest.mark.parametrize("M", [1, 4, 8])
def test_independent_linears_in_one_launch(gpu, oracle, M):
    # q / k / v style: the same activations through three weights of different widths, then two of different K
    import torch
    lib = capi.load()
    _, dom, _ = gpu
    stream = torch.cuda.Stream()
    for shapes in ([(2304, 1000), (2304, 385), (2304, 4096)], [(1057, 193), (4096, 512)], [(513, 64)]):
        ws, w, dA, dC, ref = [], [], [], [], []
        for i, (K, N) in enumerate(shapes):
            B, sw = make_weights(K, N, seed=N + i)
            A = make_activations(M, K, seed=K, dtype="f16")
            w.append(rk.Weights(dom, B, sw))
            ws.append(rk.Workspace(dom, rk.default_config(M, N, K)))
            assert ws[-1].set_schedule(5, 0) == 0              # the batch form belongs to the decode kernel
            dA.append(torch.from_numpy(A.view(np.int16)).cuda())
            dC.append(torch.full((M, N), 0x5555, dtype=torch.int16, device="cuda"))
            ref.append(oracle.linear(A, B, sw)[1])
        torch.cuda.synchronize()
        before = ws[0].launch_count()
        assert rk.enqueue_batch_f16(ws, w, dA, dC, stream.cuda_stream) == 0
        stream.synchronize()
        assert ws[0].launch_count() == before + 1                      # one launch for all of them
        for x, c, r in zip(ws, dC, ref):
            assert x.finish() == 0
            assert np.array_equal(c.cpu().numpy().view(np.uint16), r)
        # argument errors: a repeated workspace, mixed token counts
        assert rk.enqueue_batch_f16([ws[0], ws[0]], [w[0], w[0]], [dA[0], dA[0]], [dC[0], dC[0]], stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
        if M < 8:
            other = rk.Workspace(dom, rk.default_config(M + 1, shapes[0][1], shapes[0][0]))
            assert other.set_schedule(5, 0) == 0
            dA2 = torch.zeros((M + 1, shapes[0][0]), dtype=torch.int16, device="cuda")
            dC2 = torch.zeros((M + 1, shapes[0][1]), dtype=torch.int16, device="cuda")
            if len(ws) > 1:
                assert rk.enqueue_batch_f16([other, ws[1]], [w[0], w[1]], [dA2, dA[1]], [dC2, dC[1]], stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
            other.free()
        for x in ws + w:
            x.free()
