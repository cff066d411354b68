"""The benchmark configurations at full size through the C ABI, against the oracle.

Every shape a throughput figure is quoted on has a parity case here, in the regime the figure is
measured in: the 2048-token prefill linear, the fused FFN at 128 and 1024 tokens, the 70B-class FFN
at 32 and 4096 tokens and its per-GPU column shards, and problems whose tile count exceeds the
number of CTA pairs so that the persistent tensor-core kernel walks several tiles per pair.

Full CPU contractions at these sizes would take minutes, so the integer sums are checked with the
reference's own sampling for large shapes -- 17 evenly spaced columns x all rows
(src/rk_npu_w4a8_tune_data.cpp:30-33, examples/bench_w4a8.cpp:131-151), plus the columns either side
of every 256-column tile edge for the multi-tile cases -- and the epilogue over the WHOLE output:
out == dequant(int32 sums, token scales, channel scales), bit for bit.
"""
import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from oracle.harness import make_activations, make_weights, sample_columns

pytestmark = pytest.mark.gpu


def edge_columns(N, step=256, limit=96):
    cols = set(sample_columns(N).tolist())
    edges = list(range(step, N, step))
    if len(edges) > limit:
        edges = edges[:: max(1, len(edges) // limit)]
    for e in edges:
        cols.update((e - 1, e))
    cols.add(N - 1)
    return np.array(sorted(c for c in cols if 0 <= c < N), np.int32)


def check_linear(dom, oracle, M, K, N, dtype, seed, cols=None):
    """run_acc_i32 on sampled columns, then the epilogue over the whole output."""
    B, sw = make_weights(K, N, seed=seed)
    A = make_activations(M, K, seed=seed, dtype=dtype)
    if M > 2:
        A[1, :] = 0                                   # a zero row inside a large batch: scale 1, exact zeros
    half = dtype == "f16"
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    acc = np.zeros((M, N), np.int32)
    assert ws.run_acc_i32(w, A, acc) == 0
    cols = sample_columns(N) if cols is None else cols
    rc, s, inv = oracle.scales(A)
    assert rc == 0
    q = oracle.quantize(A, inv)
    assert np.array_equal(acc[:, cols], oracle.gemm_i32_columns(q, B, cols)), "int32 sums differ on the sampled columns"
    out = np.zeros((M, N), np.uint16 if half else np.float32)
    assert (ws.run_f16 if half else ws.run_f32)(w, A, out) == 0
    assert np.array_equal(bits(out), bits(oracle.dequant(acc, s, sw, half))), "epilogue differs from the exact expression"
    if M > 2:
        assert not out[1].any()
    ws.free()
    w.free()


def check_ffn(dom, oracle, M, K, F, N, seed, run_down=True):
    """Fused FFN: gate/up sums and middle on sampled features (all rows), the down projection's
    scales over all rows, its sums on sampled columns and its epilogue over the whole output."""
    Bg, sg = make_weights(K, 2 * F, seed=seed)
    A = make_activations(M, K, seed=seed, dtype="f32")
    wg = rk.Weights(dom, Bg, sg)
    gu = rk.Workspace(dom, rk.default_config(M, 2 * F, K))
    feats = sample_columns(F)
    pair_cols = np.concatenate([feats, feats + F]).astype(np.int32)
    rc, s, inv = oracle.scales(A)
    assert rc == 0
    acc_s = oracle.gemm_i32_columns(oracle.quantize(A, inv), Bg, pair_cols)
    ref_mid_s, _ = oracle.swiglu(acc_s, s, sg[pair_cols], mode=1)
    middle = np.zeros((M, F), np.float32)
    if not run_down:
        assert gu.run_swiglu_f32(wg, A, middle) == 0
        assert np.array_equal(bits(middle[:, feats]), bits(ref_mid_s)), "middle differs on the sampled features"
        gu.free()
        wg.free()
        return
    Bd, sd = make_weights(F, N, seed=seed + 1)
    wd = rk.Weights(dom, Bd, sd)
    dn = rk.Workspace(dom, rk.default_config(M, N, F))
    C = np.zeros((M, N), np.float32)
    assert rk.run_ffn_f32(gu, wg, dn, wd, A, middle, C) == 0
    assert np.array_equal(bits(middle[:, feats]), bits(ref_mid_s)), "middle differs on the sampled features"
    # the down projection quantises `middle` with scales from the collected row maxima: they must equal a rescan
    rc, s2, inv2 = oracle.scales(middle)
    assert rc == 0
    rc, got_s, _ = dn.last_quant()
    assert rc == 0 and np.array_equal(bits(got_s), bits(s2)), "reused row scales differ from a rescan of middle"
    cols = sample_columns(N)
    acc_dn = oracle.gemm_i32_columns(oracle.quantize(middle, inv2), Bd, cols)
    ref_c = oracle.dequant(acc_dn, s2, sd[cols], False)
    assert np.array_equal(bits(C[:, cols]), bits(ref_c)), "down projection differs on the sampled columns"
    # and the whole output: a plain linear on the same middle through the exact int32 entry
    acc_full = np.zeros((M, N), np.int32)
    assert dn.run_acc_i32(wd, middle, acc_full) == 0
    assert np.array_equal(acc_full[:, cols], acc_dn)
    assert np.array_equal(bits(C), bits(oracle.dequant(acc_full, s2, sd, False)))
    for x in (gu, dn, wg, wd):
        x.free()


def test_prefill_2048x4096x14336(gpu, oracle):
    _, dom, _ = gpu
    check_linear(dom, oracle, 2048, 4096, 14336, "f16", seed=2, cols=edge_columns(14336))


@pytest.mark.parametrize("M", [1, 128, 1024])
def test_ffn_4096_14336_4096(gpu, oracle, M):
    _, dom, _ = gpu
    check_ffn(dom, oracle, M, 4096, 14336, 4096, seed=30 + M)


# more tiles than CTA pairs: every pair of the persistent kernel walks two or more tiles (accumulator
# hand-over between tiles, ring wrap across tiles); ragged token and channel tails included
@pytest.mark.parametrize("shape", [(512, 1024, 20480), (300, 1024, 20481), (1100, 640, 9999)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_persistent_kernel_many_tiles_per_pair(gpu, oracle, shape, dtype):
    _, dom, _ = gpu
    M, K, N = shape
    check_linear(dom, oracle, M, K, N, dtype, seed=M + N, cols=edge_columns(N))


@pytest.mark.parametrize("shape", [(512, 1024, 10240), (300, 1057, 9984)], ids=lambda s: "x".join(map(str, s)))
def test_persistent_kernel_swiglu_many_tiles_per_pair(gpu, oracle, shape):
    _, dom, _ = gpu
    M, K, F = shape
    check_ffn(dom, oracle, M, K, F, 0, seed=M + F, run_down=False)


# 70B-class layer (hidden 8192, intermediate 28672): the whole layer on one GPU at 32 tokens and the
# column shards a GPU holds when the layer is split over 2 and 8 GPUs (gate/up feature slice, down
# column slice over the full reduction length)
def test_ffn_70b_decode_32_tokens(gpu, oracle):
    _, dom, _ = gpu
    check_ffn(dom, oracle, 32, 8192, 28672, 8192, seed=70)


@pytest.mark.parametrize("ranks", [2, 8])
def test_ffn_70b_per_gpu_shards_32_tokens(gpu, oracle, ranks):
    _, dom, _ = gpu
    check_ffn(dom, oracle, 32, 8192, 28672 // ranks, 0, seed=71 + ranks, run_down=False)
    check_linear(dom, oracle, 32, 28672, 8192 // ranks, "f32", seed=72 + ranks)


def test_ffn_70b_prefill_4096_tokens_per_gpu_shard(gpu, oracle):
    # the 8-GPU shard of the 4096-token layer; the whole layer at 4096 tokens is the same kernels on 8x the columns
    _, dom, _ = gpu
    check_ffn(dom, oracle, 4096, 8192, 28672 // 8, 0, seed=80, run_down=False)
    check_linear(dom, oracle, 4096, 28672, 1024, "f32", seed=81)
