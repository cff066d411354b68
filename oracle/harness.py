"""ctypes access to the CPU checkers and the seeded synthetic inputs.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the
benchmark's CPU legs.  The shipped package never imports this module.

Two checkers:
  * ``Oracle``     -- oracle/w4a8_oracle.c, the C restatement of the reference path.
  * ``Reference``  -- oracle/_ref/librk_npu_ref.so, the reference's own CPU stages
                      compiled from its sources plus oracle/ref_glue.cpp (present only
                      where it was built; ``Reference.available()`` says whether it is).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "_build" / "libw4a8_oracle.so"
REF_SO = HERE / "_ref" / "librk_npu_ref.so"

ERR_PARAM = -3


def build(verbose: bool = False) -> None:
    """Compile the checkers (the reference one only where its sources exist)."""
    out = subprocess.run(["make", "-C", str(HERE), "-j8"], capture_output=True, text=True)
    if out.returncode:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if verbose:
        print(out.stdout)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


class Oracle:
    """The C restatement (each routine cites the reference in w4a8_oracle.c)."""

    def __init__(self):
        if not ORACLE_SO.exists():
            build()
        self.lib = C.CDLL(str(ORACLE_SO))
        L = self.lib
        L.orc_half_to_float.restype = C.c_float
        L.orc_half_to_float.argtypes = [C.c_uint16]
        L.orc_float_to_half.restype = C.c_uint16
        L.orc_float_to_half.argtypes = [C.c_float]
        L.orc_silu_poly.restype = C.c_float
        L.orc_silu_poly.argtypes = [C.c_float]
        L.orc_silu_expf.restype = C.c_float
        L.orc_silu_expf.argtypes = [C.c_float]
        L.orc_weight_fingerprint.restype = C.c_uint64
        L.orc_weight_fingerprint.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.orc_fnv_bytes.restype = C.c_uint64
        L.orc_fnv_bytes.argtypes = [C.c_uint64, C.c_void_p, C.c_size_t]
        L.orc_moe_middle_row.restype = C.c_float
        L.orc_moe_middle_row.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_void_p]

    # ---- binary16
    def half_to_float(self, h: np.ndarray) -> np.ndarray:
        h = _c(h, np.uint16)
        out = np.empty(h.shape, np.float32)
        self.lib.orc_half_to_float_n(_ptr(h), _ptr(out), C.c_int64(h.size))
        return out

    def float_to_half(self, f: np.ndarray) -> np.ndarray:
        f = _c(f, np.float32)
        out = np.empty(f.shape, np.uint16)
        self.lib.orc_float_to_half_n(_ptr(f), _ptr(out), C.c_int64(f.size))
        return out

    # ---- stages
    def scales(self, A: np.ndarray):
        half = A.dtype == np.uint16
        A = _c(A, np.uint16 if half else np.float32)
        M, K = A.shape
        s = np.empty(M, np.float32)
        inv = np.empty(M, np.float32)
        rc = self.lib.orc_scales(_ptr(A), int(half), M, K, _ptr(s), _ptr(inv))
        return rc, s, inv

    def quantize(self, A: np.ndarray, inverse: np.ndarray) -> np.ndarray:
        half = A.dtype == np.uint16
        A = _c(A, np.uint16 if half else np.float32)
        M, K = A.shape
        q = np.empty((M, K), np.int8)
        self.lib.orc_quantize(_ptr(A), int(half), M, K, _ptr(_c(inverse, np.float32)), _ptr(q))
        return q

    def gemm_i32(self, q: np.ndarray, B: np.ndarray) -> np.ndarray:
        q = _c(q, np.int8)
        B = _c(B, np.int8)
        M, K = q.shape
        N = B.shape[1]
        acc = np.empty((M, N), np.int32)
        self.lib.orc_gemm_i32(_ptr(q), _ptr(B), M, K, N, _ptr(acc))
        return acc

    def gemm_i32_columns(self, q, B, columns) -> np.ndarray:
        q = _c(q, np.int8)
        B = _c(B, np.int8)
        cols = _c(columns, np.int32)
        M, K = q.shape
        acc = np.empty((M, cols.size), np.int32)
        self.lib.orc_gemm_i32_columns(_ptr(q), _ptr(B), M, K, B.shape[1], _ptr(cols), int(cols.size), _ptr(acc))
        return acc

    def dequant(self, acc, a_scale, w_scale, half: bool) -> np.ndarray:
        acc = _c(acc, np.int32)
        M, N = acc.shape
        out = np.empty((M, N), np.uint16 if half else np.float32)
        self.lib.orc_dequant(M, N, _ptr(acc), _ptr(_c(a_scale, np.float32)), _ptr(_c(w_scale, np.float32)),
                             int(half), _ptr(out))
        return out

    def swiglu(self, acc, a_scale, w_scale, mode: int = 1):
        acc = _c(acc, np.int32)
        M, N = acc.shape
        F = N // 2
        middle = np.empty((M, F), np.float32)
        maxima = np.empty(M, np.uint32)
        self.lib.orc_swiglu(M, F, _ptr(acc), _ptr(_c(a_scale, np.float32)), _ptr(_c(w_scale, np.float32)),
                            mode, _ptr(middle), _ptr(maxima))
        return middle, maxima

    def finish_scales(self, maxima):
        maxima = _c(maxima, np.uint32)
        M = maxima.size
        s = np.empty(M, np.float32)
        inv = np.empty(M, np.float32)
        rc = self.lib.orc_finish_scales(M, _ptr(maxima), _ptr(s), _ptr(inv))
        return rc, s, inv

    def linear(self, A, B, w_scale):
        """Returns (rc, out, acc int32, scales)."""
        half = A.dtype == np.uint16
        A = _c(A, np.uint16 if half else np.float32)
        B = _c(B, np.int8)
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), np.uint16 if half else np.float32)
        acc = np.empty((M, N), np.int32)
        s = np.empty(M, np.float32)
        rc = self.lib.orc_linear(_ptr(A), int(half), M, K, N, _ptr(B), _ptr(_c(w_scale, np.float32)),
                                 _ptr(out), _ptr(acc), _ptr(s))
        return rc, out, acc, s

    def w8_linear(self, A, B, w_scale, a_scale=None):
        """One typed W8A8 linear (dynamic scales, or the caller's static ones).  Returns dict(rc, out, acc, scales, codes)."""
        half = A.dtype == np.uint16
        A = _c(A, np.uint16 if half else np.float32)
        B = _c(B, np.int8)
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), np.uint16 if half else np.float32)
        acc = np.empty((M, N), np.int32)
        s = np.empty(M, np.float32)
        q = np.empty((M, K), np.int8)
        static = None if a_scale is None else _c(a_scale, np.float32)
        rc = getattr(self.lib, 'orc_w8_linear')(_ptr(A), int(half), M, K, N, _ptr(B), _ptr(_c(w_scale, np.float32)), _ptr(static),
                                               _ptr(out), _ptr(acc), _ptr(s), _ptr(q))
        return dict(rc=rc, out=out, acc=acc, scales=s, codes=q)

    # ---- routed experts
    def moe_quantize_rows(self, X, validate: bool = True):
        """Nearest-even row quantisation of the routed operator.  Returns (rc, codes, scales); rc 1: a row was rejected."""
        X = _c(X, np.float32)
        rows, n = X.shape
        q = np.zeros((rows, n), np.int8)
        s = np.zeros(rows, np.float32)
        rc = 0
        for r in range(rows):
            one = C.c_float(0)
            rc |= self.lib.orc_moe_quantize_row(_ptr(X[r]), n, int(validate), _ptr(q[r]), C.byref(one))
            s[r] = one.value
        return rc, q, s

    def moe_middle_row(self, acc, input_scale, w_scale, mode: int = 1):
        """acc: [2I] int32 sums, gate then up.  Returns (scale, codes[I])."""
        acc = _c(acc, np.int32)
        I = acc.shape[0] // 2
        q = np.zeros(I, np.int8)
        scale = self.lib.orc_moe_middle_row(_ptr(acc), I, C.c_float(input_scale), _ptr(_c(w_scale, np.float32)), mode, _ptr(q))
        return float(scale), q

    def moe_run(self, experts, shared: int, top: int, codes, row_scales, ids, routes, mode: int = 1):
        """experts: dict(gate_up [E,H,2I] int8, gate_up_scales [E,2I], down [E,I,H] int8, down_scales [E,H]), the
        shared expert last when shared == 1.  Returns (rc, out [rows,H] fp32)."""
        G = _c(experts["gate_up"], np.int8)
        D = _c(experts["down"], np.int8)
        E, H, I2 = G.shape
        codes = _c(codes, np.int8)
        rows = codes.shape[0]
        out = np.zeros((rows, H), np.float32)
        rc = self.lib.orc_moe_run(rows, H, I2 // 2, E - shared, shared, top, _ptr(G), _ptr(_c(experts["gate_up_scales"], np.float32)),
                                  _ptr(D), _ptr(_c(experts["down_scales"], np.float32)), _ptr(codes),
                                  _ptr(_c(row_scales, np.float32)), _ptr(_c(ids, np.int32)), _ptr(_c(routes, np.float32)), mode,
                                  _ptr(out))
        return rc, out

    def add_rmsnorm_f16(self, x, residual, gamma, eps: float = 1.0e-5):
        """x, residual: [M, D] fp16 bit patterns (row-major); gamma: [D].  Returns (residual_out, norm_out) bit patterns."""
        x, residual, gamma = _c(x, np.uint16), _c(residual, np.uint16), _c(gamma, np.uint16)
        M, D = x.shape
        sums, norm = np.zeros((M, D), np.uint16), np.zeros((M, D), np.uint16)
        self.lib.orc_add_rmsnorm_f16(M, D, C.c_float(eps), _ptr(x), _ptr(residual), _ptr(gamma), _ptr(sums), _ptr(norm))
        return sums, norm

    def ffn(self, A, B_gu, s_gu, B_dn, s_dn, mode: int = 1):
        """Returns dict(rc, middle, C, acc_gate_up, acc_down, scales_down_in)."""
        A = _c(A, np.float32)
        B_gu = _c(B_gu, np.int8)
        B_dn = _c(B_dn, np.int8)
        M, K = A.shape
        F = B_gu.shape[1] // 2
        N = B_dn.shape[1]
        middle = np.zeros((M, F), np.float32)
        Cc = np.zeros((M, N), np.float32)
        a1 = np.zeros((M, 2 * F), np.int32)
        a2 = np.zeros((M, N), np.int32)
        sd = np.zeros(M, np.float32)
        rc = self.lib.orc_ffn(_ptr(A), M, K, F, N, _ptr(B_gu), _ptr(_c(s_gu, np.float32)), _ptr(B_dn),
                              _ptr(_c(s_dn, np.float32)), mode, _ptr(middle), _ptr(Cc), _ptr(a1), _ptr(a2), _ptr(sd))
        return dict(rc=rc, middle=middle, C=Cc, acc_gate_up=a1, acc_down=a2, scales_down_in=sd)

    def weight_check(self, B, w_scale):
        B = _c(B, np.int8)
        K, N = B.shape
        corr = np.empty(N, np.int32)
        rc = self.lib.orc_weight_check(K, N, _ptr(B), _ptr(_c(w_scale, np.float32)), _ptr(corr))
        return rc, corr

    def bound(self, B, requested: int = 0, fallback: int = 0):
        B = _c(B, np.int8)
        K, N = B.shape
        kt = C.c_int(0)
        pos = C.c_int64(0)
        neg = C.c_int64(0)
        mask = C.c_uint64(0)
        rc = self.lib.orc_bound_i4_weights(K, N, _ptr(B), requested, fallback, C.byref(kt), C.byref(pos),
                                           C.byref(neg), C.byref(mask))
        return rc, kt.value, pos.value, neg.value, mask.value

    def fingerprint(self, B, w_scale) -> int:
        B = _c(B, np.int8)
        K, N = B.shape
        return int(self.lib.orc_weight_fingerprint(K, N, _ptr(B), _ptr(_c(w_scale, np.float32))))


class Reference:
    """The reference's own CPU stages (built from its sources by oracle/Makefile)."""

    @staticmethod
    def available() -> bool:
        return REF_SO.exists()

    def __init__(self):
        if not REF_SO.exists():
            raise RuntimeError("reference checker not built (oracle/_ref/librk_npu_ref.so)")
        self.lib = C.CDLL(str(REF_SO))
        L = self.lib
        L.ref_fingerprint.restype = C.c_uint64
        L.ref_half_to_float.restype = C.c_float
        L.ref_half_to_float.argtypes = [C.c_uint16]
        L.ref_float_to_half.restype = C.c_uint16
        L.ref_float_to_half.argtypes = [C.c_float]
        L.ref_layer_create.restype = C.c_void_p
        L.ref_layer_free.argtypes = [C.c_void_p]
        if hasattr(L, "ref_moe_middle_row"):
            L.ref_moe_middle_row.restype = C.c_float
            L.ref_moe_middle_row.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_void_p]

    def host_threads(self) -> int:
        return int(self.lib.ref_host_threads())

    def half_to_float(self, h: np.ndarray) -> np.ndarray:
        h = _c(h, np.uint16)
        out = np.empty(h.shape, np.float32)
        self.lib.ref_half_to_float_n(_ptr(h), _ptr(out), C.c_int64(h.size))
        return out

    def float_to_half(self, f: np.ndarray) -> np.ndarray:
        f = _c(f, np.float32)
        out = np.empty(f.shape, np.uint16)
        self.lib.ref_float_to_half_n(_ptr(f), _ptr(out), C.c_int64(f.size))
        return out

    def quantize(self, A, threads: int = 1):
        half = A.dtype == np.uint16
        A = _c(A, np.uint16 if half else np.float32)
        M, K = A.shape
        s = np.empty(M, np.float32)
        inv = np.empty(M, np.float32)
        q = np.zeros((M, K), np.int8)
        rc = self.lib.ref_quantize(_ptr(A), int(half), M, K, threads, _ptr(s), _ptr(inv), _ptr(q))
        return rc, s, inv, q

    def linear(self, A, B, w_scale, k_tile=480, m_tile=64, n_tile=1024, mask=1, threads=4, want_acc=True):
        half = A.dtype == np.uint16
        A = _c(A, np.uint16 if half else np.float32)
        B = _c(B, np.int8)
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), np.uint16 if half else np.float32)
        acc = np.zeros((M, N), np.int32) if want_acc else None
        s = np.empty(M, np.float32)
        sat = C.c_int64(0)
        stage = (C.c_double * 4)()
        prep = C.c_double(0)
        rc = self.lib.ref_linear(_ptr(A), int(half), M, K, N, _ptr(B), _ptr(_c(w_scale, np.float32)), k_tile,
                                 m_tile, n_tile, C.c_uint(mask), threads, _ptr(out), _ptr(acc), _ptr(s),
                                 C.byref(sat), stage, C.byref(prep))
        return dict(rc=rc, out=out, acc=acc, scales=s, saturated=sat.value, stage_us=list(stage),
                    prepare_us=prep.value)

    def w8_linear(self, A, B, w_scale, a_scale=None):
        """One typed W8A8 linear (dynamic scales, or the caller's static ones).  Returns dict(rc, out, acc, scales, codes)."""
        half = A.dtype == np.uint16
        A = _c(A, np.uint16 if half else np.float32)
        B = _c(B, np.int8)
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), np.uint16 if half else np.float32)
        acc = np.empty((M, N), np.int32)
        s = np.empty(M, np.float32)
        q = np.empty((M, K), np.int8)
        static = None if a_scale is None else _c(a_scale, np.float32)
        rc = getattr(self.lib, 'ref_w8_linear')(_ptr(A), int(half), M, K, N, _ptr(B), _ptr(_c(w_scale, np.float32)), _ptr(static),
                                               _ptr(out), _ptr(acc), _ptr(s), _ptr(q))
        return dict(rc=rc, out=out, acc=acc, scales=s, codes=q)

    def k_partition_query(self, M, K, k_tile) -> int:
        return int(self.lib.ref_k_partition_query(M, K, k_tile))

    def moe_middle_row(self, acc, input_scale, w_scale):
        """The reference's fused middle stage of the routed operator on one row (its x86 build: std::exp)."""
        acc = _c(acc, np.int32)
        I = acc.shape[0] // 2
        q = np.zeros(I, np.int8)
        scale = self.lib.ref_moe_middle_row(_ptr(acc), I, C.c_float(input_scale), _ptr(_c(w_scale, np.float32)), _ptr(q))
        return float(scale), q

    def layer(self, B, w_scale, k_tile=480):
        B = _c(B, np.int8)
        K, N = B.shape
        h = self.lib.ref_layer_create(K, N, k_tile, _ptr(B), _ptr(_c(w_scale, np.float32)))
        if not h:
            raise RuntimeError("reference layer preparation failed")
        return C.c_void_p(h), (K, N)

    def layer_run(self, handle, shape, A, m_tile=64, n_tile=1024, mask=1, threads=4):
        half = A.dtype == np.uint16
        A = _c(A, np.uint16 if half else np.float32)
        M = A.shape[0]
        out = np.empty((M, shape[1]), np.uint16 if half else np.float32)
        stage = (C.c_double * 4)()
        rc = self.lib.ref_layer_run(handle, _ptr(A), int(half), M, m_tile, n_tile, C.c_uint(mask), threads,
                                    _ptr(out), stage)
        return rc, out, list(stage)

    def layer_free(self, handle):
        self.lib.ref_layer_free(handle)

    def ffn(self, A, B_gu, s_gu, B_dn, s_dn, kt_gu=480, kt_dn=480, m_tile=64, n_tile=1024, mask=1, threads=4,
            swiglu_only=False):
        A = _c(A, np.float32)
        B_gu = _c(B_gu, np.int8)
        M, K = A.shape
        F = B_gu.shape[1] // 2
        middle = np.zeros((M, F), np.float32)
        if swiglu_only:
            B_dn = np.zeros((F, 1), np.int8)
            s_dn = np.ones(1, np.float32)
        B_dn = _c(B_dn, np.int8)
        N = B_dn.shape[1]
        Cc = np.zeros((M, N), np.float32)
        sd = np.zeros(M, np.float32)
        sat = C.c_int64(0)
        stage = (C.c_double * 4)()
        rc = self.lib.ref_ffn(_ptr(A), M, K, F, N, _ptr(B_gu), _ptr(_c(s_gu, np.float32)), _ptr(B_dn),
                              _ptr(_c(s_dn, np.float32)), kt_gu, kt_dn, m_tile, n_tile, C.c_uint(mask), threads,
                              int(swiglu_only), _ptr(middle), _ptr(Cc), _ptr(sd), C.byref(sat), stage)
        return dict(rc=rc, middle=middle, C=Cc, scales_down_in=sd, saturated=sat.value, stage_us=list(stage))

    def bound(self, B, requested=0, fallback=0):
        B = _c(B, np.int8)
        K, N = B.shape
        kt = C.c_int(0)
        pos = C.c_int64(0)
        neg = C.c_int64(0)
        mask = C.c_uint64(0)
        rc = self.lib.ref_bound(K, N, _ptr(B), requested, fallback, C.byref(kt), C.byref(pos), C.byref(neg),
                                C.byref(mask))
        return rc, kt.value, pos.value, neg.value, mask.value

    def dequant(self, acc, a_scale, w_scale, half, threads=1):
        acc = _c(acc, np.int32)
        M, N = acc.shape
        out = np.empty((M, N), np.uint16 if half else np.float32)
        self.lib.ref_dequant(M, N, _ptr(acc), _ptr(_c(a_scale, np.float32)), _ptr(_c(w_scale, np.float32)),
                             int(half), _ptr(out), threads)
        return out

    def finish_scales(self, maxima):
        maxima = _c(maxima, np.uint32)
        M = maxima.size
        s = np.empty(M, np.float32)
        inv = np.empty(M, np.float32)
        rc = self.lib.ref_finish_scales(M, 1, _ptr(maxima), M, _ptr(s), _ptr(inv))
        return rc, s, inv

    def fingerprint(self, B, w_scale) -> int:
        B = _c(B, np.int8)
        K, N = B.shape
        return int(self.lib.ref_fingerprint(K, N, _ptr(B), _ptr(_c(w_scale, np.float32))))


# --------------------------------------------------------------------- inputs
# The seeded synthetic tensors (the benchmark configurations' value distributions) live in the package, where bench.py and the
# profiler workloads use them too; they are re-exported here for the tests.
from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights, sample_columns  # noqa: E402,F401
