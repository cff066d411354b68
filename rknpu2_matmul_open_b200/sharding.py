"""Column sharding of one W4A8 linear over the ranks of a torch.distributed group.

The reference splits the output columns of a GEMM over its NPU cores in contiguous runs of
64-column blocks, the first ``blocks % cores`` cores taking one block more
(src/rk_npu_i4_plan.cpp:37-43).  The same partition is used over GPUs: every rank holds the
weight columns of its run and computes C[:, n0:n1]; per-column arithmetic is unchanged, so the
assembled result is bit-identical for any number of ranks.  The only exchange is the
all-gather that reassembles the output where a caller needs all of it.
"""
from __future__ import annotations

import numpy as np


def shard_columns(N: int, world: int, rank: int) -> tuple[int, int]:
    """[n0, n1) of `rank`; empty for ranks beyond the number of 64-column blocks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a group of {world}")
    blocks = (N + 63) // 64
    start = 0
    for r in range(world):
        count = blocks // world + (1 if r < blocks % world else 0)
        if r == rank:
            return min(N, start * 64), min(N, (start + count) * 64)
        start += count
    raise AssertionError


def shard_weights(B: np.ndarray, w_scale: np.ndarray, world: int, rank: int):
    """This rank's slice of B[K,N] codes and w_scale[N]."""
    n0, n1 = shard_columns(B.shape[1], world, rank)
    return np.ascontiguousarray(B[:, n0:n1]), np.ascontiguousarray(w_scale[n0:n1]), (n0, n1)


def shard_ffn_weights(B_gate_up: np.ndarray, scale_gate_up: np.ndarray, world: int, rank: int):
    """Gate and up are sharded by the SAME feature slice so that SwiGLU stays local:
    returns the re-packed [gate(f0:f1), up(f0:f1)] columns, their scales and (f0, f1)."""
    F = B_gate_up.shape[1] // 2
    f0, f1 = shard_columns(F, world, rank)
    cols = np.r_[f0:f1, F + f0:F + f1]
    return np.ascontiguousarray(B_gate_up[:, cols]), np.ascontiguousarray(scale_gate_up[cols]), (f0, f1)


def gather_columns(local, N: int, group=None):
    """All-gather row-major [M, n1-n0] shards into the full [M, N] tensor on every rank.
    Shards differ in width, so each is padded to the widest before the collective."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    M = local.shape[0]
    widths = [shard_columns(N, world, r) for r in range(world)]
    pad = max(b - a for a, b in widths)
    send = torch.zeros((M, pad), dtype=local.dtype, device=local.device)
    send[:, : local.shape[1]] = local
    recv = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(recv, send, group=group)
    out = torch.empty((M, N), dtype=local.dtype, device=local.device)
    for (a, b), part in zip(widths, recv):
        out[:, a:b] = part[:, : b - a]
    return out
