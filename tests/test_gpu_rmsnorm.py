"""CUDA residual add + RMSNorm through the C ABI against the oracle, bit for bit on both outputs: the original's
blocking call on caller-owned buffers in its block-8 layout (its two validated shapes and others), the enqueue form
on device tensors in both layouts, every rejection of the run call in the original's order, buffer accounting."""
import ctypes as C

import numpy as np
import pytest

from rknpu2_matmul_open_b200 import capi, rmsnorm
from test_rmsnorm_oracle import board_inputs

pytestmark = pytest.mark.gpu


def buffers(domain, count, size):
    return [rmsnorm.Buffer(domain, size) for _ in range(count)]


@pytest.mark.parametrize("M,D,eps", [(1, 4096, 1e-5), (128, 4096, 1e-5),       # the original's validated programs
                                     (3, 64, 1e-6), (37, 8192, 1e-5), (256, 1024, 1e-5), (5, 32768, 1e-5), (33, 40, 0.5),
                                     (130, 5120, 1e-5), (2, 8, 1e-5)])
def test_blocking_run_equals_the_oracle(gpu, oracle, M, D, eps):
    ctx, d0, _ = gpu
    x, r, g = board_inputs(M, D, 7 * M + D)
    if M > 2:
        x[2], r[2] = 0, 0                                    # a zero row normalises to zeros
        x[0, : D // 2] = np.float16(60000).view(np.uint16)   # large values: the sum of squares needs its range
    cfg = rmsnorm.default_config(M, D)
    cfg.eps = eps
    plan = rmsnorm.AddRmsNormPlan(d0, cfg, g)
    bx, br, bs, bn = buffers(d0, 4, rmsnorm.query(cfg).tensor_bytes)
    bx.array()[:] = rmsnorm.to_block8(x)
    br.array()[:] = rmsnorm.to_block8(r)
    for _ in range(2):                                       # twice: nothing is left over from a run
        bs.array()[:] = 0xFFFF
        bn.array()[:] = 0xFFFF
        assert plan.run(bx, br, bs, bn) == capi.RK_NPU_OK
        want_sums, want_norm = oracle.add_rmsnorm_f16(x, r, g, eps)
        assert np.array_equal(rmsnorm.from_block8(bs.array(), M, D), want_sums)
        assert np.array_equal(rmsnorm.from_block8(bn.array(), M, D), want_norm)
    assert np.array_equal(bx.array(), rmsnorm.to_block8(x)) and np.array_equal(br.array(), rmsnorm.to_block8(r))
    for b in (bx, br, bs, bn):
        assert b.free() == capi.RK_NPU_OK
    plan.free()


@pytest.mark.parametrize("M,D,rows", [(1, 4096, 1), (128, 4096, 128), (128, 4096, 77), (1024, 8192, 1024), (64, 2048, 9),
                                      (300, 12288, 300)])
@pytest.mark.parametrize("row_major", [False, True])
def test_enqueue_on_device_tensors_equals_the_oracle(gpu, oracle, M, D, rows, row_major):
    import torch
    ctx, d0, _ = gpu
    x, r, g = board_inputs(rows, D, 3 * M + D + rows)
    plan = rmsnorm.AddRmsNormPlan(d0, rmsnorm.default_config(M, D), g)
    lay = (lambda a: a) if row_major else rmsnorm.to_block8
    dx = torch.from_numpy(lay(x).astype(np.int16)).cuda()
    dr = torch.from_numpy(lay(r).astype(np.int16)).cuda()
    ds, dn = torch.full_like(dx, -1), torch.full_like(dx, -1)
    stream = torch.cuda.current_stream()
    assert plan.enqueue(rows, row_major, dx.data_ptr(), dr.data_ptr(), ds.data_ptr(), dn.data_ptr(), stream.cuda_stream) == capi.RK_NPU_OK
    stream.synchronize()
    want_sums, want_norm = oracle.add_rmsnorm_f16(x, r, g)
    got_sums, got_norm = ds.cpu().numpy().view(np.uint16), dn.cpu().numpy().view(np.uint16)
    if not row_major:
        got_sums, got_norm = rmsnorm.from_block8(got_sums, rows, D), rmsnorm.from_block8(got_norm, rows, D)
    assert np.array_equal(got_sums.reshape(rows, D), want_sums)
    assert np.array_equal(got_norm.reshape(rows, D), want_norm)
    # rejections: too many rows, a bad layout flag, a misaligned tensor, an output on top of an input
    p = (dx.data_ptr(), dr.data_ptr(), ds.data_ptr(), dn.data_ptr())
    assert plan.enqueue(M + 1, row_major, *p, stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
    assert plan.enqueue(0, row_major, *p, stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
    assert plan.enqueue(rows, 2, *p, stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
    assert plan.enqueue(rows, row_major, p[0] + 2, p[1], p[2], p[3], stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
    assert plan.enqueue(rows, row_major, p[0], p[1], p[0], p[3], stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
    assert plan.enqueue(rows, row_major, p[0], p[1], p[2], p[2] + 16, stream.cuda_stream) == capi.RK_NPU_ERR_PARAM
    plan.free()


def test_outputs_outside_the_normal_fp16_range(gpu, oracle):
    # gamma of 60000 overflows the normalised value to infinity, gamma near 2^-14 and below makes it subnormal or zero:
    # the kernel's single-precision shortcut must hand all of these to the defining double-precision expression
    import torch
    ctx, d0, _ = gpu
    M, D = 6, 512
    rng = np.random.default_rng(77)
    x = rng.normal(0, 1, (M, D)) * np.array([1, 1e-3, 2000, 1, 30, 1e-2])[:, None]
    r = rng.normal(0, 0.3, (M, D)) * np.array([1, 1e-3, 100, 0, 1, 1e-4])[:, None]
    g = np.tile(np.array([60000, 6.1e-5, 1, 3e-6, 0.5, 6e-8, -2, 0], np.float64), D // 8)
    x, r, g = (a.astype(np.float16).view(np.uint16) for a in (x, r, g))
    want_sums, want_norm = oracle.add_rmsnorm_f16(x, r, g)
    out = want_norm.view(np.float16)
    assert np.isinf(out).any() and ((out != 0) & (np.abs(out) < 6.1e-5)).any() and (out == 0).any() and not np.isnan(out).any()
    plan = rmsnorm.AddRmsNormPlan(d0, rmsnorm.default_config(M, D), g)
    for row_major in (False, True):
        lay = (lambda a: a) if row_major else rmsnorm.to_block8
        dx, dr = (torch.from_numpy(lay(a).astype(np.int16)).cuda() for a in (x, r))
        ds, dn = torch.zeros_like(dx), torch.zeros_like(dx)
        assert plan.enqueue(M, row_major, dx.data_ptr(), dr.data_ptr(), ds.data_ptr(), dn.data_ptr(), 0) == capi.RK_NPU_OK
        torch.cuda.synchronize()
        got_s, got_n = ds.cpu().numpy().view(np.uint16), dn.cpu().numpy().view(np.uint16)
        if not row_major:
            got_s, got_n = rmsnorm.from_block8(got_s, M, D), rmsnorm.from_block8(got_n, M, D)
        assert np.array_equal(got_s.reshape(M, D), want_sums) and np.array_equal(got_n.reshape(M, D), want_norm)
    plan.free()


def test_rejections_follow_the_original_order(gpu, lib):
    ctx, d0, d1 = gpu
    M, D = 4, 64
    _, _, g = board_inputs(M, D, 1)
    cfg = rmsnorm.default_config(M, D)
    plan = rmsnorm.AddRmsNormPlan(d0, cfg, g)
    size = M * D * 2
    bx, br, bs, bn = buffers(d0, 4, size)
    small, foreign = rmsnorm.Buffer(d0, size - 2), rmsnorm.Buffer(d1, size)
    big = rmsnorm.Buffer(d0, 3 * size)
    for b in (bx, br):
        b.array()[:] = 0
    bs.array()[:] = 0x1234
    bn.array()[:] = 0x1234
    run = lambda a, b, c, d: plan.run(a, b, c, d)
    assert run(small, br, bs, bn) == capi.RK_NPU_ERR_NOMEM          # src/rk_npu_add_rmsnorm_f16.cpp:279
    assert run(bx, br, bs, foreign) == capi.RK_NPU_ERR_DOMAIN        # :280
    assert run(small, br, bs, foreign) == capi.RK_NPU_ERR_NOMEM      # in argument order
    assert run(bx, br, bx, bn) == capi.RK_NPU_ERR_PARAM              # :282-284 overlaps
    assert run(bx, br, bs, bs) == capi.RK_NPU_ERR_PARAM
    assert run(bx, br, br, bn) == capi.RK_NPU_ERR_PARAM
    stale = capi.Mem.from_buffer_copy(bx.mem)
    stale.ctx_id += 1
    assert lib.rk_npu_add_rmsnorm_f16_run(ctx.handle, plan.handle, C.byref(stale), C.byref(br.mem), C.byref(bs.mem),
                                          C.byref(bn.mem)) == capi.RK_NPU_ERR_NOMEM        # a buffer of another context
    assert lib.rk_npu_add_rmsnorm_f16_run(ctx.handle, plan.handle, None, C.byref(br.mem), C.byref(bs.mem), C.byref(bn.mem)) == capi.RK_NPU_ERR_PARAM
    assert np.all(bs.array() == 0x1234) and np.all(bn.array() == 0x1234)      # nothing was written

    # views: two halves of one allocation are distinct tensors; overlapping views are refused
    va, vb, vc = capi.Mem(), capi.Mem(), capi.Mem()
    assert lib.rk_npu_mem_view(C.byref(big.mem), 0, size, C.byref(va)) == capi.RK_NPU_OK
    assert lib.rk_npu_mem_view(C.byref(big.mem), size, size, C.byref(vb)) == capi.RK_NPU_OK
    assert lib.rk_npu_mem_view(C.byref(big.mem), size + 16, size, C.byref(vc)) == capi.RK_NPU_OK
    call = lambda out_s, out_n: lib.rk_npu_add_rmsnorm_f16_run(ctx.handle, plan.handle, C.byref(bx.mem), C.byref(br.mem), C.byref(out_s), C.byref(out_n))
    assert call(va, vb) == capi.RK_NPU_OK
    assert call(vb, vc) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_sync(ctx.handle, C.byref(va), 1) == capi.RK_NPU_OK
    assert lib.rk_npu_mem_sync(ctx.handle, C.byref(va), 2) == capi.RK_NPU_OK
    assert lib.rk_npu_mem_sync(ctx.handle, C.byref(va), 3) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_mem_free(ctx.handle, C.byref(va)) == capi.RK_NPU_OK and va.size == 0 and big.mem.handle != 0     # a view only clears

    # freeing: a copy of a freed struct is refused, not freed twice
    copy = capi.Mem.from_buffer_copy(small.mem)
    assert small.free() == capi.RK_NPU_OK and small.mem.vaddr is None
    assert lib.rk_npu_mem_free(ctx.handle, C.byref(copy)) == capi.RK_NPU_ERR_PARAM
    for b in (bx, br, bs, bn, foreign, big):
        assert b.free() == capi.RK_NPU_OK
    plan.free()


def test_buffers_are_accounted_to_their_domain(gpu):
    ctx, d0, _ = gpu
    before = d0.memory_stats()
    b = rmsnorm.Buffer(d0, 1 << 20, capi.RK_NPU_MEM_CACHEABLE if hasattr(capi, "RK_NPU_MEM_CACHEABLE") else 2)
    during = d0.memory_stats()
    assert during.live_bytes == before.live_bytes + (1 << 20) and during.creates == before.creates + 1
    assert b.mem.flags == (1 << 0) | (1 << 3) | (1 << 4) and b.mem.size == b.mem.capacity == 1 << 20 and b.mem.dma_addr % 256 == 0
    b.array(np.uint8)[:] = 5
    assert b.free() == capi.RK_NPU_OK
    after = d0.memory_stats()
    assert after.live_bytes == before.live_bytes and after.destroys == before.destroys + 1
