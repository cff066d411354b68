"""Host-side mirror of the residual add + RMSNorm operator (include/rknpu_b200_rmsnorm.h) and of the caller-owned
buffers it works on (rk_npu_mem_*), over the C ABI.  All compute happens in the CUDA library.

``Buffer`` wraps one rk_npu_mem (page-locked host memory the GPU addresses directly; ``array`` is a numpy view of the
host mapping).  ``AddRmsNormPlan`` wraps rk_npu_add_rmsnorm_f16_plan: ``run`` is the original's blocking call on four
buffers in its block-8 layout, ``enqueue`` the form on device tensors and the caller's stream.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .capi import AddRmsNormConfig, AddRmsNormSizes, Mem
from .w4a8 import W4A8Error


def to_block8(rows: np.ndarray) -> np.ndarray:
    """[M, D] -> the original's (D/8, M, 8) order, flattened."""
    M, D = rows.shape
    return np.ascontiguousarray(rows.reshape(M, D // 8, 8).transpose(1, 0, 2)).reshape(-1)


def from_block8(flat: np.ndarray, M: int, D: int) -> np.ndarray:
    """The inverse of to_block8."""
    return np.ascontiguousarray(np.asarray(flat).reshape(D // 8, M, 8).transpose(1, 0, 2)).reshape(M, D)


class Buffer:
    """rk_npu_mem_alloc / rk_npu_mem_free."""

    def __init__(self, domain, size: int, flags: int = 0):
        self.lib = capi.load()
        self.ctx = domain.ctx
        self.mem = Mem()
        rc = self.lib.rk_npu_mem_alloc(domain.handle, size, flags, C.byref(self.mem))
        if rc != capi.RK_NPU_OK:
            raise W4A8Error(rc, "rk_npu_mem_alloc")

    def array(self, dtype=np.uint16) -> np.ndarray:
        """The host mapping as a numpy array (valid until free())."""
        count = self.mem.size // np.dtype(dtype).itemsize
        return np.ctypeslib.as_array(C.cast(self.mem.vaddr, C.POINTER(C.c_uint8)), (self.mem.size,)).view(dtype)[:count]

    def free(self) -> int:
        rc = capi.RK_NPU_OK
        if self.mem.handle:
            rc = self.lib.rk_npu_mem_free(self.ctx.handle, C.byref(self.mem))
        return rc


def default_config(M: int, D: int) -> AddRmsNormConfig:
    """rk_npu_add_rmsnorm_f16_config_init"""
    c = AddRmsNormConfig()
    capi.load().rk_npu_add_rmsnorm_f16_config_init(C.byref(c), M, D)
    return c


def query(config: AddRmsNormConfig) -> AddRmsNormSizes:
    """rk_npu_add_rmsnorm_f16_query"""
    sizes = AddRmsNormSizes()
    rc = capi.load().rk_npu_add_rmsnorm_f16_query(C.byref(config), C.byref(sizes))
    if rc != capi.RK_NPU_OK:
        raise W4A8Error(rc, "rk_npu_add_rmsnorm_f16_query")
    return sizes


class AddRmsNormPlan:
    """rk_npu_add_rmsnorm_f16_plan_create / _run / _plan_free; gamma: [D] fp16 bit patterns."""

    def __init__(self, domain, config: AddRmsNormConfig, gamma):
        self.lib = capi.load()
        self.ctx = domain.ctx
        self.config = config
        gamma = np.ascontiguousarray(gamma, np.uint16)
        self.handle = self.lib.rk_npu_add_rmsnorm_f16_plan_create(domain.handle, C.byref(config), gamma.ctypes.data_as(C.c_void_p))
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_PARAM, "rk_npu_add_rmsnorm_f16_plan_create")

    def run(self, x: Buffer, residual: Buffer, residual_out: Buffer, norm_out: Buffer, ctx=None) -> int:
        """The blocking call; returns the C return code."""
        return self.lib.rk_npu_add_rmsnorm_f16_run((ctx or self.ctx).handle, self.handle, C.byref(x.mem), C.byref(residual.mem),
                                                   C.byref(residual_out.mem), C.byref(norm_out.mem))

    def enqueue(self, rows: int, row_major: bool, x: int, residual: int, residual_out: int, norm_out: int, stream: int = 0) -> int:
        """rk_npu_b200_add_rmsnorm_f16_enqueue on device addresses; returns the C return code."""
        return self.lib.rk_npu_b200_add_rmsnorm_f16_enqueue(self.handle, rows, int(row_major), x, residual, residual_out, norm_out, stream)

    def free(self):
        if self.handle:
            self.lib.rk_npu_add_rmsnorm_f16_plan_free(self.handle)
            self.handle = None
