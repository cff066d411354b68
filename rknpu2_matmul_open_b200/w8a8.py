"""Host-side mirror of the typed W8A8 operators (include/rknpu_b200_quant.h) over the C ABI.

``MatmulWeights`` wraps rk_npu_{i8i8i32,f16i8f16,f32i8f32}_weights, ``MatmulWorkspace`` wraps
rk_npu_matmul_workspace (made from an rk_npu_matmul_strategy, fixed to one exact M and operator kind); the run
methods have the argument meaning and return codes of the C calls.  All compute happens in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import capi
from .capi import MatmulStrategy, MatmulWeightConfig
from .w4a8 import W4A8Error, _ptr

I8I8I32, F16_DYNAMIC, F16_STATIC, F32_DYNAMIC, F32_STATIC = range(5)
_FAMILY = {I8I8I32: "i8i8i32", F16_DYNAMIC: "f16i8f16", F16_STATIC: "f16i8f16", F32_DYNAMIC: "f32i8f32", F32_STATIC: "f32i8f32"}


def default_strategy(kind: int, M: int, N: int, K: int, k_tile: int | None = None) -> MatmulStrategy:
    """A valid strategy for (kind, M, N, K): one K wave, one device core, the first permitted CPU."""
    s = MatmulStrategy()
    s.op_kind, s.M, s.N, s.K = kind, M, N, K
    s.k_tile = k_tile or K
    s.n_tile = min(3072, (N + 31) // 32 * 32)
    s.a_layout = 0
    s.wave_count = (K + s.k_tile - 1) // s.k_tile
    s.n_groups = ((N + 31) // 32 * 32 + s.n_tile - 1) // s.n_tile
    s.npu_core_mask = 1
    cpu = min(c for c in os.sched_getaffinity(0) if c < 64)
    s.cpu_core_mask = 1 << cpu
    s.cpu_threads = 1
    s.c_layout = 0
    return s


class MatmulWeights:
    """rk_npu_<family>_weights_create / _free.  `family`: 'i8i8i32' (no scales), 'f16i8f16' or 'f32i8f32'."""

    def __init__(self, domain, family: str, B: np.ndarray, w_scale: np.ndarray | None = None, k_tile: int | None = None,
                 compress: bool = False):
        """compress: the *_weights_create_compress constructor (the same object in this library)."""
        self.lib = capi.load()
        self.family = family
        B = np.ascontiguousarray(B, np.int8)
        K, N = B.shape
        self.config = MatmulWeightConfig(K, N, k_tile or K)
        create = getattr(self.lib, f"rk_npu_{family}_weights_create" + ("_compress" if compress else ""))
        if family == "i8i8i32":
            self.handle = create(domain.handle, C.byref(self.config), _ptr(B))
        else:
            w_scale = np.ascontiguousarray(w_scale, np.float32)
            self.handle = create(domain.handle, C.byref(self.config), _ptr(B), _ptr(w_scale))
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_PARAM, f"rk_npu_{family}_weights_create")

    def free(self):
        if self.handle:
            getattr(self.lib, f"rk_npu_{self.family}_weights_free")(self.handle)
            self.handle = None


class MatmulWorkspace:
    """rk_npu_matmul_workspace_create / _free and the blocking runs."""

    def __init__(self, domain, strategy: MatmulStrategy):
        self.lib = capi.load()
        self.strategy = strategy
        self.handle = self.lib.rk_npu_matmul_workspace_create(domain.handle, C.byref(strategy))
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_PARAM, "rk_npu_matmul_workspace_create")

    def run_i8(self, w: MatmulWeights, A, out) -> int:
        return self.lib.rk_npu_i8i8i32_run(self.handle, w.handle, _ptr(A), _ptr(out))

    def run_dynamic(self, w: MatmulWeights, A, out) -> int:
        return getattr(self.lib, f"rk_npu_{w.family}_run_dynamic")(self.handle, w.handle, _ptr(A), _ptr(out))

    def run_static(self, w: MatmulWeights, A, a_scale, out) -> int:
        return getattr(self.lib, f"rk_npu_{w.family}_run_static")(self.handle, w.handle, _ptr(A), _ptr(a_scale), _ptr(out))

    def launch_count(self) -> int:
        return self.lib.rk_npu_b200_matmul_launch_count(self.handle)

    def free(self):
        if self.handle:
            self.lib.rk_npu_matmul_workspace_free(self.handle)
            self.handle = None
