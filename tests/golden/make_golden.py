"""Generate tests/golden/*.npz from the REFERENCE's own CPU stages.

Run where oracle/_ref/librk_npu_ref.so has been built (the reference tree present):

    python tests/golden/make_golden.py

Every fixture stores its inputs as well as the reference's outputs, so it does not
depend on a random-number generator's version.  Outputs come from the reference's
compiled code (scales, quantise + pack, reconstruction, dequantise, SwiGLU, scale
finishing) around the CPU stand-in for its device step (oracle/ref_glue.cpp).
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle.harness import Reference, make_activations, make_weights  # noqa: E402

OUT = Path(__file__).resolve().parent


def uniform_codes(K, N, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(-8, 8, size=(K, N), dtype=np.int8)


def power_scales(N):
    return np.ldexp(np.float32(1), -(np.arange(N) % 6 + 6)).astype(np.float32)


def ramp_activations(M, K, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    A = (rng.integers(0, 2049, size=(M, K)) - 1024).astype(np.float32)
    A *= np.ldexp(np.float32(1), (np.arange(M) % 5 - 8))[:, None].astype(np.float32)
    if M > 1:
        A[0, :] = 0   # zero row: scale must be 1 and the output exactly 0
    return A


def main():
    ref = Reference()
    linear = {}
    # (M, K, N, k_tile, kind): tail shapes from the reference's own board tests
    cases = [(1, 1, 1, 480, "ramp"), (3, 33, 65, 480, "ramp"), (5, 1025, 129, 480, "ramp"), (7, 513, 257, 256, "ramp"),
             (2, 480, 64, 480, "extreme"), (5, 1025, 129, 480, "extreme"), (2, 20003, 65, 480, "extreme"),
             (16, 2048, 256, 480, "normal"), (9, 1057, 193, 480, "normal"), (33, 1057, 257, 2048, "normal")]
    for i, (M, K, N, kt, kind) in enumerate(cases):
        if kind == "normal":
            B, sw = make_weights(K, N, seed=100 + i)
            A32 = make_activations(M, K, seed=100 + i, dtype="f32")
        elif kind == "ramp":
            B, sw, A32 = uniform_codes(K, N, 200 + i), power_scales(N), ramp_activations(M, K, 300 + i)
        else:
            B = np.where((np.arange(K * N) % N % 2).reshape(K, N) == 1, 7, -8).astype(np.int8)
            sw = power_scales(N)
            A32 = np.where((np.arange(M) % 2)[:, None] == 1, np.float32(127), np.float32(-127)) * np.ones((1, K), np.float32)
        A16 = ref.float_to_half(A32)
        r32 = ref.linear(A32, B, sw, k_tile=kt, m_tile=3, n_tile=128, mask=1, threads=1)
        r16 = ref.linear(A16, B, sw, k_tile=kt, m_tile=3, n_tile=128, mask=1, threads=1)
        assert r32["rc"] == 0 and r16["rc"] == 0 and r32["saturated"] == 0 and r16["saturated"] == 0, (M, K, N)
        _, s32, _, q32 = ref.quantize(A32)
        _, s16, _, q16 = ref.quantize(A16)
        tag = f"c{i}"
        linear.update({f"{tag}_shape": np.array([M, K, N, kt]), f"{tag}_B": B, f"{tag}_sw": sw, f"{tag}_A32": A32,
                       f"{tag}_A16": A16, f"{tag}_out32": r32["out"], f"{tag}_out16": r16["out"],
                       f"{tag}_acc32": r32["acc"], f"{tag}_acc16": r16["acc"], f"{tag}_s32": s32, f"{tag}_s16": s16,
                       f"{tag}_q32": q32, f"{tag}_q16": q16})
    linear["count"] = np.array(len(cases))
    np.savez_compressed(OUT / "linear_reference.npz", **linear)

    ffn = {}
    ffn_cases = [(1, 479, 96, 192), (9, 959, 128, 192), (17, 545, 992, 192), (8, 1024, 256, 320)]
    for i, (M, K, F, N) in enumerate(ffn_cases):
        Bg, sg = make_weights(K, 2 * F, seed=400 + i)
        Bd, sd = make_weights(F, N, seed=500 + i)
        A = make_activations(M, K, seed=400 + i, dtype="f32")
        r = ref.ffn(A, Bg, sg, Bd, sd, kt_gu=480, kt_dn=480, m_tile=16, n_tile=256, mask=1, threads=2)
        assert r["rc"] == 0 and r["saturated"] == 0
        tag = f"f{i}"
        ffn.update({f"{tag}_shape": np.array([M, K, F, N]), f"{tag}_Bg": Bg, f"{tag}_sg": sg, f"{tag}_Bd": Bd,
                    f"{tag}_sd": sd, f"{tag}_A": A, f"{tag}_middle": r["middle"], f"{tag}_C": r["C"],
                    f"{tag}_scales_down": r["scales_down_in"]})
    ffn["count"] = np.array(len(ffn_cases))
    np.savez_compressed(OUT / "ffn_reference.npz", **ffn)

    # binary16 conversion tables from the reference's header-only routines
    halves = np.arange(65536, dtype=np.uint16)
    floats = np.arange(0, 2 ** 32, 65521, dtype=np.uint64).astype(np.uint32).view(np.float32)
    np.savez_compressed(OUT / "half_reference.npz", h2f=ref.half_to_float(halves).view(np.uint32), f_in=floats.view(np.uint32),
                        f2h=ref.float_to_half(floats))
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
