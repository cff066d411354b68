"""Host-side mirror of the rk_npu_w4a8 operator interface over the C ABI.

Object names follow the C handles: a ``Context`` (rk_npu_ctx) owns ``Domain``s
(rk_npu_iommu_domain); ``Weights`` (rk_npu_w4a8_weights) and ``Workspace``
(rk_npu_w4a8_workspace) are created from a domain and the run methods have the argument
meaning and return codes of rk_npu_w4a8_run_f32 / _f16 / _swiglu_f32 / _ffn_f32.
Tensors may be numpy arrays (host memory, the original contract) or torch CUDA tensors
(device memory, no copies).  All compute happens in the CUDA library; nothing here
touches tensor values.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .capi import (RK_NPU_OK, I4WeightConfig, W4A8Config, W4A8FfnTimings, W4A8MemoryInfoEx, W4A8Options, W4A8Timings,
                   W4A8WeightInfo)


class W4A8Error(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        lib = capi.load()
        super().__init__(f"{what}: {lib.rk_npu_strerror(code).decode()} ({code})")


def _ptr(t):
    """Raw address of a numpy array or a torch tensor (host or device)."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        if not t.flags["C_CONTIGUOUS"]:
            raise ValueError("tensor must be compact row-major")
        return C.c_void_p(t.ctypes.data)
    if hasattr(t, "data_ptr"):
        if not t.is_contiguous():
            raise ValueError("tensor must be compact row-major")
        return C.c_void_p(t.data_ptr())
    raise TypeError(f"unsupported tensor type {type(t)}")


class Context:
    """rk_npu_open / rk_npu_close. dev: None (current CUDA device) or 'cuda:N'."""

    def __init__(self, dev: str | None = None):
        self.lib = capi.load()
        self.handle = self.lib.rk_npu_open(dev.encode() if dev else None)
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_OPEN, f"rk_npu_open({dev!r})")

    @classmethod
    def open_group(cls, dev: str, rank: int, world: int, group_id: bytes) -> "Context":
        """rk_npu_b200_open_group: this process is `rank` of `world` GPUs sharing the 128-byte id rank 0 obtained from
        rk_npu_b200_group_id; weights are column-sharded and results all-gathered inside the library."""
        self = cls.__new__(cls)
        self.lib = capi.load()
        ident = (C.c_ubyte * 128).from_buffer_copy(bytes(group_id))
        self.handle = self.lib.rk_npu_b200_open_group(dev.encode(), rank, world, ident)
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_OPEN, f"rk_npu_b200_open_group({dev!r}, {rank}, {world})")
        return self

    @property
    def device(self) -> int:
        return self.lib.rk_npu_b200_device(self.handle)

    def all_gather(self, dBuffer, bytes_per_rank: int, stream: int = 0) -> int:
        """rk_npu_b200_group_all_gather: in-place all-gather of the group (every rank's piece at its slot)."""
        return self.lib.rk_npu_b200_group_all_gather(self.handle, _ptr(dBuffer), bytes_per_rank, C.c_void_p(stream))

    def domain(self, domain_id: int = 0) -> "Domain":
        return Domain(self, domain_id)

    def close(self):
        if self.handle:
            self.lib.rk_npu_close(self.handle)
            self.handle = None


class Domain:
    def __init__(self, ctx: Context, domain_id: int):
        self.ctx = ctx
        self.lib = ctx.lib
        self.handle = self.lib.rk_npu_iommu_domain_create(ctx.handle, domain_id)
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_DOMAIN, f"rk_npu_iommu_domain_create({domain_id})")

    def memory_stats(self) -> capi.DomainMemoryStats:
        s = capi.DomainMemoryStats()
        self.lib.rk_npu_iommu_domain_memory_stats(self.handle, C.byref(s))
        return s

    def free(self):
        if self.handle:
            self.lib.rk_npu_iommu_domain_free(self.handle)
            self.handle = None


def default_config(M: int, N: int, K: int, **overrides) -> W4A8Config:
    cfg = W4A8Config()
    capi.load().rk_npu_w4a8_config_init(C.byref(cfg), M, N, K)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def memory_query(cfg: W4A8Config, options: W4A8Options | None = None):
    info = W4A8MemoryInfoEx()
    rc = capi.load().rk_npu_w4a8_memory_query_ex(C.byref(cfg), C.byref(options) if options is not None else None,
                                                 C.byref(info))
    return rc, info


class Weights:
    """rk_npu_w4a8_weights_create: B[K,N] int8 codes in [-8,7], w_scale[N] fp32 > 0."""

    def __init__(self, domain: Domain, B: np.ndarray, w_scale: np.ndarray, k_tile: int = 480):
        self.lib = domain.lib
        B = np.ascontiguousarray(B, dtype=np.int8)
        w_scale = np.ascontiguousarray(w_scale, dtype=np.float32)
        self.K, self.N = B.shape
        key = I4WeightConfig(self.K, self.N, k_tile)
        self.handle = self.lib.rk_npu_w4a8_weights_create(domain.handle, C.byref(key), _ptr(B), _ptr(w_scale))
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_PARAM, "rk_npu_w4a8_weights_create")
        self.domain = domain

    def info(self) -> W4A8WeightInfo:
        out = W4A8WeightInfo()
        self.lib.rk_npu_w4a8_weights_query(self.handle, C.byref(out))
        return out

    @property
    def k_tile(self) -> int:
        return self.info().config.k_tile

    def free(self):
        if self.handle:
            self.lib.rk_npu_w4a8_weights_free(self.handle)
            self.handle = None


class Workspace:
    """rk_npu_w4a8_workspace_create[_ex]: fixed (M, N, K, k_tile); owns all scratch."""

    def __init__(self, domain: Domain, cfg: W4A8Config, options: W4A8Options | None = None):
        self.lib = domain.lib
        self.cfg = cfg
        self.handle = self.lib.rk_npu_w4a8_workspace_create_ex(domain.handle, C.byref(cfg),
                                                               C.byref(options) if options is not None else None)
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_PARAM, "rk_npu_w4a8_workspace_create_ex")
        self.domain = domain

    # ---- blocking calls (return the C status code; timings optional)
    def run_f32(self, weights: Weights, A, C_out, timings: W4A8Timings | None = None) -> int:
        return self.lib.rk_npu_w4a8_run_f32(self.handle, weights.handle, _ptr(A), _ptr(C_out),
                                            C.byref(timings) if timings is not None else None)

    def run_f16(self, weights: Weights, A, C_out, timings: W4A8Timings | None = None) -> int:
        return self.lib.rk_npu_w4a8_run_f16(self.handle, weights.handle, _ptr(A), _ptr(C_out),
                                            C.byref(timings) if timings is not None else None)

    def run_swiglu_f32(self, weights: Weights, A, middle, timings: W4A8Timings | None = None) -> int:
        return self.lib.rk_npu_w4a8_run_swiglu_f32(self.handle, weights.handle, _ptr(A), _ptr(middle),
                                                   C.byref(timings) if timings is not None else None)

    def run_acc_i32(self, weights: Weights, A, acc) -> int:
        half = (A.dtype == np.uint16) if isinstance(A, np.ndarray) else (A.element_size() == 2)
        return self.lib.rk_npu_b200_w4a8_run_acc_i32(self.handle, weights.handle, _ptr(A), int(half), _ptr(acc))

    def last_quant(self):
        s = np.empty(self.cfg.M, np.float32)
        q = np.empty((self.cfg.M, self.cfg.K), np.int8)
        rc = self.lib.rk_npu_b200_w4a8_last_quant(self.handle, _ptr(s), _ptr(q))
        return rc, s, q

    # ---- enqueue forms (device tensors, caller's stream)
    def enqueue_f16(self, weights: Weights, dA, dC, stream: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_enqueue_f16(self.handle, weights.handle, _ptr(dA), _ptr(dC), C.c_void_p(stream))

    def enqueue_f32(self, weights: Weights, dA, dC, stream: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_enqueue_f32(self.handle, weights.handle, _ptr(dA), _ptr(dC), C.c_void_p(stream))

    def enqueue_swiglu_f32(self, weights: Weights, dA, dMiddle, stream: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_enqueue_swiglu_f32(self.handle, weights.handle, _ptr(dA), _ptr(dMiddle),
                                                            C.c_void_p(stream))

    # ---- column-sharded FFN: the pieces around the exchange between GPUs (rknpu_b200_ext.h)
    def enqueue_swiglu_collect_f32(self, weights: Weights, dA, dMiddle, dRowMaxima, stream: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_enqueue_swiglu_collect_f32(self.handle, weights.handle, _ptr(dA), _ptr(dMiddle),
                                                                    _ptr(dRowMaxima), C.c_void_p(stream))

    def enqueue_quantize_slice(self, dMiddle, dRowMaxima, dCodes, stream: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_enqueue_quantize_slice(self.handle, _ptr(dMiddle), _ptr(dRowMaxima), _ptr(dCodes),
                                                                C.c_void_p(stream))

    def enqueue_codes_f32(self, weights: Weights, dCodes, parts: int, dRowMaxima, dC, stream: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_enqueue_codes_f32(self.handle, weights.handle, _ptr(dCodes), int(parts),
                                                           _ptr(dRowMaxima), _ptr(dC), C.c_void_p(stream))

    # ---- group of GPUs: this rank's columns only, no exchange
    def shard(self):
        """(two_range, n0, n1, columns) of the columns this rank computes."""
        v = [C.c_int() for _ in range(4)]
        self.lib.rk_npu_b200_w4a8_workspace_shard(self.handle, *[C.byref(x) for x in v])
        return bool(v[0].value), v[1].value, v[2].value, v[3].value

    def enqueue_local_f16(self, weights: Weights, dA, dLocal, stream: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_enqueue_local_f16(self.handle, weights.handle, _ptr(dA), _ptr(dLocal), C.c_void_p(stream))

    def enqueue_local_f32(self, weights: Weights, dA, dLocal, stream: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_enqueue_local_f32(self.handle, weights.handle, _ptr(dA), _ptr(dLocal), C.c_void_p(stream))

    def finish(self) -> int:
        return self.lib.rk_npu_b200_w4a8_finish(self.handle)

    def set_schedule(self, variant: int = 0, split_k: int = 0) -> int:
        return self.lib.rk_npu_b200_w4a8_set_schedule(self.handle, variant, split_k)

    def schedule(self) -> tuple[int, int]:
        """(kernel family, cooperating CTAs per column tile or 0 = automatic) this workspace runs."""
        v, k = C.c_int(0), C.c_int(0)
        self.lib.rk_npu_b200_w4a8_schedule(self.handle, C.byref(v), C.byref(k))
        return v.value, k.value

    def launch_count(self) -> int:
        return int(self.lib.rk_npu_b200_w4a8_launch_count(self.handle))

    def free(self):
        if self.handle:
            self.lib.rk_npu_w4a8_workspace_free(self.handle)
            self.handle = None


def run_ffn_f32(gate_up: Workspace, gate_up_weights: Weights, down: Workspace, down_weights: Weights, A, middle, C_out,
                timings: W4A8FfnTimings | None = None) -> int:
    """rk_npu_w4a8_run_ffn_f32: gate/up -> SwiGLU -> down with row-scale reuse (blocking)."""
    return gate_up.lib.rk_npu_w4a8_run_ffn_f32(gate_up.handle, gate_up_weights.handle, down.handle, down_weights.handle,
                                               _ptr(A), _ptr(middle), _ptr(C_out),
                                               C.byref(timings) if timings is not None else None)


def enqueue_batch_f16(workspaces, weights, dAs, dLocals, stream: int = 0) -> int:
    """rk_npu_b200_w4a8_enqueue_batch_f16: up to four independent decode linears (same token count) in one launch."""
    n = len(workspaces)
    arr = lambda items: (C.c_void_p * n)(*[x if isinstance(x, C.c_void_p) else C.c_void_p(x) for x in items])
    return workspaces[0].lib.rk_npu_b200_w4a8_enqueue_batch_f16(
        n, arr([w.handle for w in workspaces]), arr([w.handle for w in weights]), arr([_ptr(a) for a in dAs]),
        arr([_ptr(c) for c in dLocals]), C.c_void_p(stream))


def enqueue_ffn_f32(gate_up: Workspace, gate_up_weights: Weights, down: Workspace, down_weights: Weights, dA, dMiddle,
                    dC, stream: int = 0) -> int:
    return gate_up.lib.rk_npu_b200_w4a8_enqueue_ffn_f32(gate_up.handle, gate_up_weights.handle, down.handle,
                                                        down_weights.handle, _ptr(dA), _ptr(dMiddle), _ptr(dC),
                                                        C.c_void_p(stream))


__all__ = ["Context", "Domain", "Weights", "Workspace", "W4A8Error", "default_config", "memory_query", "run_ffn_f32",
           "enqueue_ffn_f32", "enqueue_batch_f16", "RK_NPU_OK"]
