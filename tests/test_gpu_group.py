"""A group of GPUs behind the ordinary interface: one process per GPU opens rk_npu_b200_open_group, passes the
FULL weights and activations to the unchanged reference calls, and every rank must end up with the full
result, bit for bit what the oracle computes for one device (column sharding changes no arithmetic).

Covered: plain linears (binary16 and fp32, contiguous and two-range shards, uneven block counts, ragged N),
the fused FFN with all-reduced row maxima, NaN rejection on every rank, and the enqueue form on device tensors.
Skipped where fewer than two GPUs are visible; the partition rule itself is tested on the CPU."""
import ctypes as C

import numpy as np
import pytest


def _free_all(*objs):
    for o in objs:
        o.free()


def _rank_main(rank, world, group_id, cases, queue):
    try:
        _rank_body(rank, world, group_id, cases, queue)
    except BaseException as exc:   # noqa: BLE001
        import traceback
        queue.put(("error", rank, f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
        raise


def _rank_body(rank, world, group_id, cases, queue):
    import torch

    import rknpu2_matmul_open_b200 as rk
    from rknpu2_matmul_open_b200 import capi
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights

    torch.cuda.set_device(rank)
    ctx = rk.Context.open_group(f"cuda:{rank}", rank, world, group_id)
    lib = capi.load()
    assert lib.rk_npu_b200_group_rank(ctx.handle) == rank and lib.rk_npu_b200_group_size(ctx.handle) == world
    dom = ctx.domain(0)
    results = []
    for (M, K, F, N) in cases:
        # plain linear, both types, full tensors on every rank
        B, sw = make_weights(K, N, seed=5)
        w = rk.Weights(dom, B, sw)
        ws = rk.Workspace(dom, rk.default_config(M, N, K))
        A16 = make_activations(M, K, seed=5, dtype="f16")
        out16 = np.zeros((M, N), np.uint16)
        assert ws.run_f16(w, A16, out16) == 0
        A32 = make_activations(M, K, seed=6, dtype="f32")
        out32 = np.zeros((M, N), np.float32)
        assert ws.run_f32(w, A32, out32) == 0
        bad = A32.copy()
        bad[M - 1, 3] = np.nan
        assert ws.run_f32(w, bad, np.zeros((M, N), np.float32)) == capi.RK_NPU_ERR_PARAM
        # enqueue form on device tensors
        dA = torch.from_numpy(A16.view(np.int16)).cuda()
        dC = torch.zeros((M, N), dtype=torch.int16, device="cuda")
        s = torch.cuda.current_stream()
        assert ws.enqueue_f16(w, dA, dC, s.cuda_stream) == 0
        torch.cuda.synchronize()
        assert ws.finish() == 0
        dev16 = dC.cpu().numpy().view(np.uint16)
        _free_all(ws, w)
        # fused FFN (gate/up columns N % 128 == 0 so that SwiGLU pairs stay on one GPU)
        ffn = None
        if F:
            Bg, sg = make_weights(K, 2 * F, seed=7)
            Bd, sd = make_weights(F, N, seed=8)
            wg, wd = rk.Weights(dom, Bg, sg), rk.Weights(dom, Bd, sd)
            gu = rk.Workspace(dom, rk.default_config(M, 2 * F, K))
            dn = rk.Workspace(dom, rk.default_config(M, N, F))
            middle, Cc = np.zeros((M, F), np.float32), np.zeros((M, N), np.float32)
            assert rk.run_ffn_f32(gu, wg, dn, wd, A32, middle, Cc) == 0
            only = np.zeros((M, F), np.float32)
            assert gu.run_swiglu_f32(wg, A32, only) == 0 and np.array_equal(only.view(np.uint32), middle.view(np.uint32))
            ffn = (middle, Cc)
            _free_all(gu, dn, wg, wd)
        results.append((out16, out32, dev16, ffn))
    queue.put(("ok", rank, results))
    dom.free()
    ctx.close()


@pytest.mark.gpu
def test_group_context_matches_one_device_bit_for_bit(oracle):
    import torch
    import torch.multiprocessing as mp

    from rknpu2_matmul_open_b200 import capi
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    lib = capi.load()
    ident = (C.c_ubyte * 128)()
    assert lib.rk_npu_b200_group_id(ident) == 0
    # (M, K, F, N): F = 0 skips the FFN; N = 1000 is ragged and contiguous-sharded, 1152 two-range, 4160 = 65 blocks (uneven)
    cases = [(8, 1057, 1024, 1152), (40, 2304, 0, 1000), (3, 513, 0, 4160), (160, 1024, 640, 512)]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, bytes(ident), cases, queue), daemon=True) for r in range(world)]
    got = {}
    try:
        for p in procs:
            p.start()
        for _ in range(world):
            item = queue.get(timeout=600)
            assert item[0] == "ok", f"rank {item[1]} failed: {item[2]}"
            got[item[1]] = item[2]
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    for i, (M, K, F, N) in enumerate(cases):
        B, sw = make_weights(K, N, seed=5)
        A16 = make_activations(M, K, seed=5, dtype="f16")
        A32 = make_activations(M, K, seed=6, dtype="f32")
        ref16 = oracle.linear(A16, B, sw)[1]
        ref32 = oracle.linear(A32, B, sw)[1]
        ref_ffn = None
        if F:
            Bg, sg = make_weights(K, 2 * F, seed=7)
            Bd, sd = make_weights(F, N, seed=8)
            ref_ffn = oracle.ffn(A32, Bg, sg, Bd, sd, mode=1)
        for rank in range(world):                      # EVERY rank holds the full, exact result
            out16, out32, dev16, ffn = got[rank][i]
            assert np.array_equal(out16, ref16), (rank, i)
            assert np.array_equal(out32.view(np.uint32), ref32.view(np.uint32)), (rank, i)
            assert np.array_equal(dev16, ref16), (rank, i)
            if F:
                assert np.array_equal(ffn[0].view(np.uint32), ref_ffn["middle"].view(np.uint32)), (rank, i)
                assert np.array_equal(ffn[1].view(np.uint32), ref_ffn["C"].view(np.uint32)), (rank, i)


def test_partition_rule_is_the_reference_core_split():
    # contiguous 64-column blocks, the first blocks % world ranks one more (src/rk_npu_i4_plan.cpp:37-43)
    from rknpu2_matmul_open_b200 import capi
    from rknpu2_matmul_open_b200.sharding import shard_columns
    lib = capi.load()
    n0, n1 = C.c_int(), C.c_int()
    for N in (1, 64, 65, 193, 1000, 4096, 4160, 11008, 14336):
        for world in (1, 2, 3, 4, 8):
            covered = 0
            for rank in range(world):
                assert lib.rk_npu_b200_shard_columns(N, world, rank, C.byref(n0), C.byref(n1)) == 0
                assert (n0.value, n1.value) == shard_columns(N, world, rank)
                assert n0.value == covered or n0.value == n1.value == N
                covered = max(covered, n1.value)
            assert covered == N
    assert lib.rk_npu_b200_shard_columns(64, 2, 2, C.byref(n0), C.byref(n1)) == capi.RK_NPU_ERR_PARAM


def test_a_refused_communicator_fails_on_the_host(monkeypatch):
    # a rank that cannot join (lost peer, failed bootstrap) is told so by open_group, before any GPU work
    from rknpu2_matmul_open_b200 import capi
    lib = capi.load()
    monkeypatch.setenv("RK_NPU_B200_REFUSE_GROUP", "1")
    ident = (C.c_ubyte * 128)()
    assert not lib.rk_npu_b200_open_group(b"cuda:0", 0, 2, ident)
    assert not lib.rk_npu_b200_open_group(b"cuda:0", 2, 2, ident)      # rank outside the group: refused as an argument error
