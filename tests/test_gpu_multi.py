"""Column sharding over several GPUs of one box: one process per GPU, NCCL all-gather of the shard
outputs, assembled result compared bit for bit with the oracle.  Skipped where fewer than two GPUs
are visible (the gloo tests cover the host logic on CPU)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, shape, out_queue):
    """Child process body: any exception goes to the parent through the queue so it fails fast."""
    try:
        _rank_body(rank, world, port, shape, out_queue)
    except BaseException as exc:   # noqa: BLE001 -- reported, then the process ends
        import traceback
        out_queue.put(("error", rank, f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
        raise


def _rank_body(rank: int, world: int, port: int, shape, out_queue):
    import datetime

    import torch
    import torch.distributed as dist

    import rknpu2_matmul_open_b200 as rk
    from rknpu2_matmul_open_b200.sharding import gather_columns, shard_ffn_weights, shard_weights
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # a short collective timeout: a rank that died makes the others' next collective fail instead of waiting
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    M, K, F, N = shape
    ctx = rk.Context(f"cuda:{rank}")
    dom = ctx.domain(0)
    stream = torch.cuda.current_stream(dev)
    # plain linear, binary16
    B, sw = make_weights(K, N, seed=5)
    A = make_activations(M, K, seed=5, dtype="f16")
    Bs, ss, (n0, n1) = shard_weights(B, sw, world, rank)
    w = rk.Weights(dom, Bs, ss)
    ws = rk.Workspace(dom, rk.default_config(M, n1 - n0, K))
    dA = torch.from_numpy(A.view(np.int16)).to(dev)
    dC = torch.zeros((M, n1 - n0), dtype=torch.float16, device=dev)
    assert ws.enqueue_f16(w, dA, dC, stream.cuda_stream) == 0
    full = gather_columns(dC, N)
    # FFN: gate/up sharded by feature slice, fp32 middle gathered, down sharded by output columns
    Bg, sg = make_weights(K, 2 * F, seed=6)
    Bd, sd = make_weights(F, N, seed=7)
    A32 = make_activations(M, K, seed=6, dtype="f32")
    Bg_s, sg_s, (f0, f1) = shard_ffn_weights(Bg, sg, world, rank)
    Bd_s, sd_s, (m0, m1) = shard_weights(Bd, sd, world, rank)
    wg, wd = rk.Weights(dom, Bg_s, sg_s), rk.Weights(dom, Bd_s, sd_s)
    gu = rk.Workspace(dom, rk.default_config(M, 2 * (f1 - f0), K))
    dn = rk.Workspace(dom, rk.default_config(M, m1 - m0, F))
    dA32 = torch.from_numpy(A32).to(dev)
    dMid = torch.zeros((M, f1 - f0), dtype=torch.float32, device=dev)
    dOut = torch.zeros((M, m1 - m0), dtype=torch.float32, device=dev)
    assert gu.enqueue_swiglu_f32(wg, dA32, dMid, stream.cuda_stream) == 0
    middle = gather_columns(dMid, F)
    assert dn.enqueue_f32(wd, middle, dOut, stream.cuda_stream) == 0
    ffn = gather_columns(dOut, N)
    torch.cuda.synchronize()
    assert ws.finish() == 0 and gu.finish() == 0 and dn.finish() == 0
    # the same FFN exchanging int8 codes instead of the fp32 middle (equal feature slices only)
    ffn_codes = None
    if (F // 64) % world == 0 and F % 64 == 0:
        pc = f1 - f0
        maxima = torch.zeros(M, dtype=torch.int32, device=dev)
        codes = torch.empty((M, pc), dtype=torch.int8, device=dev)
        parts = torch.empty((world, M, pc), dtype=torch.int8, device=dev)
        dOut.zero_()
        assert gu.enqueue_swiglu_collect_f32(wg, dA32, dMid, maxima, stream.cuda_stream) == 0
        dist.all_reduce(maxima, op=dist.ReduceOp.MAX)
        assert gu.enqueue_quantize_slice(dMid, maxima, codes, stream.cuda_stream) == 0
        dist.all_gather_into_tensor(parts, codes)
        assert dn.enqueue_codes_f32(wd, parts, world, maxima, dOut, stream.cuda_stream) == 0
        ffn_codes = gather_columns(dOut, N)
        torch.cuda.synchronize()
        assert gu.finish() == 0 and dn.finish() == 0
        ffn_codes = ffn_codes.cpu().numpy()
    if rank == 0:
        out_queue.put(("ok", full.cpu().numpy().view(np.uint16), middle.cpu().numpy(), ffn.cpu().numpy(), ffn_codes))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("shape", [(8, 1057, 992, 1000), (40, 2304, 1600, 385), (33, 1057, 1024, 512)], ids=lambda s: "x".join(map(str, s)))
def test_sharded_linear_and_ffn_are_bit_exact(oracle, shape):
    import torch
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights

    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, shape, queue), daemon=True) for r in range(world)]
    try:
        for p in procs:
            p.start()
        got = queue.get(timeout=300)
        assert got[0] == "ok", f"rank {got[1]} failed: {got[2]}"
        got = got[1:]
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        # whatever happened, no child stays behind on a GPU
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    M, K, F, N = shape
    B, sw = make_weights(K, N, seed=5)
    A = make_activations(M, K, seed=5, dtype="f16")
    rc, ref, _, _ = oracle.linear(A, B, sw)
    assert rc == 0 and np.array_equal(got[0], ref)
    Bg, sg = make_weights(K, 2 * F, seed=6)
    Bd, sd = make_weights(F, N, seed=7)
    A32 = make_activations(M, K, seed=6, dtype="f32")
    ref_ffn = oracle.ffn(A32, Bg, sg, Bd, sd, mode=1)
    assert np.array_equal(got[1].view(np.uint32), ref_ffn["middle"].view(np.uint32))
    assert np.array_equal(got[2].view(np.uint32), ref_ffn["C"].view(np.uint32))
    if (F // 64) % world == 0 and F % 64 == 0:
        assert got[3] is not None and np.array_equal(got[3].view(np.uint32), ref_ffn["C"].view(np.uint32))
