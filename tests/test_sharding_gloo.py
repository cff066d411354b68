"""Column sharding over ranks (host logic), run as real torch.distributed processes on the
CPU with the gloo backend.  The per-rank linear is computed by the oracle here -- the test is
about the partition and the reassembly, which are the same code the GPU ranks use."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    from oracle.harness import Oracle, make_activations, make_weights
    from rknpu2_matmul_open_b200.sharding import gather_columns, shard_ffn_weights, shard_weights

    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle = Oracle()
    ok = True
    for (M, K, N) in [(5, 257, 1025), (3, 96, 64), (8, 512, 4096 + 64)]:
        B, sw = make_weights(K, N, seed=N)
        A = make_activations(M, K, seed=N, dtype="f32")
        Bs, ss, (n0, n1) = shard_weights(B, sw, world, rank)
        if n1 > n0:
            local = oracle.linear(A, Bs, ss)[1]
        else:
            local = np.zeros((M, 0), np.float32)
        full = gather_columns(torch.from_numpy(local), N).numpy()
        ref = oracle.linear(A, B, sw)[1]
        ok &= bool(np.array_equal(full.view(np.uint32), ref.view(np.uint32)))
    # FFN: same feature slice of gate and up per rank -> SwiGLU local, row maxima reduced with max
    M, K, F = 4, 256, 320
    Bg, sg = make_weights(K, 2 * F, seed=1)
    A = make_activations(M, K, seed=1, dtype="f32")
    Bl, sl, (f0, f1) = shard_ffn_weights(Bg, sg, world, rank)
    _, s, inv = oracle.scales(A)
    acc = oracle.gemm_i32(oracle.quantize(A, inv), Bl)
    middle_local, maxima = oracle.swiglu(acc, s, sl, mode=1)
    t = torch.from_numpy(maxima.astype(np.int64))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    middle = gather_columns(torch.from_numpy(middle_local), F).numpy()
    acc_full = oracle.gemm_i32(oracle.quantize(A, inv), Bg)
    ref_mid, ref_max = oracle.swiglu(acc_full, s, sg, mode=1)
    ok &= bool(np.array_equal(middle.view(np.uint32), ref_mid.view(np.uint32)))
    ok &= bool(np.array_equal(t.numpy().astype(np.uint32), ref_max))
    # FFN with equal feature slices: the ranks agree on the row maxima (integer max of the bit patterns), quantise
    # their own slice with the combined scale, all-gather int8 codes as [ranks][M][F/ranks], and run the
    # column-sharded down projection on them -- the protocol of the GPU path, arithmetic by the oracle.
    M, K, F, N = 5, 160, 384, 192
    Bg, sg = make_weights(K, 2 * F, seed=2)
    Bd, sd = make_weights(F, N, seed=3)
    A = make_activations(M, K, seed=2, dtype="f32")
    Bl, sl, (f0, f1) = shard_ffn_weights(Bg, sg, world, rank)
    _, s, inv = oracle.scales(A)
    middle_local, maxima = oracle.swiglu(oracle.gemm_i32(oracle.quantize(A, inv), Bl), s, sl, mode=1)
    t = torch.from_numpy(maxima.view(np.int32).copy())
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    rc, s_mid, inv_mid = oracle.finish_scales(t.numpy().view(np.uint32))
    codes = torch.from_numpy(oracle.quantize(middle_local, inv_mid))
    parts = [torch.empty_like(codes) for _ in range(world)]
    dist.all_gather(parts, codes)
    gathered = torch.stack(parts).numpy()                                   # [ranks][M][F/ranks]
    codes_full = np.ascontiguousarray(gathered.transpose(1, 0, 2).reshape(M, F))
    Bd_l, sd_l, (n0, n1) = shard_weights(Bd, sd, world, rank)
    out_local = oracle.dequant(oracle.gemm_i32(codes_full, Bd_l), s_mid, sd_l, half=False)
    out = gather_columns(torch.from_numpy(out_local), N).numpy()
    ref = oracle.ffn(A, Bg, sg, Bd, sd, mode=1)
    ok &= rc == 0 and ref["rc"] == 0
    ok &= bool(np.array_equal(s_mid.view(np.uint32), ref["scales_down_in"].view(np.uint32)))
    ok &= bool(np.array_equal(out.view(np.uint32), ref["C"].view(np.uint32)))
    Path(tmp, f"rank{rank}.ok").write_text("1" if ok else "0")
    dist.destroy_process_group()


def test_partition_is_the_reference_core_split():
    from rknpu2_matmul_open_b200.sharding import shard_columns
    # 11008 columns = 172 blocks over 8 ranks: 22,22,22,22,21,21,21,21 blocks
    widths = [shard_columns(11008, 8, r) for r in range(8)]
    assert [b - a for a, b in widths] == [1408] * 4 + [1344] * 4
    assert widths[0][0] == 0 and widths[-1][1] == 11008
    assert all(widths[i][1] == widths[i + 1][0] for i in range(7))
    assert shard_columns(65, 3, 0) == (0, 64) and shard_columns(65, 3, 1) == (64, 65) and shard_columns(65, 3, 2) == (65, 65)
    with pytest.raises(ValueError):
        shard_columns(64, 2, 2)


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_linear_and_ffn_reassemble_exactly(world, tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 1000 + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert [Path(tmp_path, f"rank{r}.ok").read_text() for r in range(world)] == ["1"] * world
