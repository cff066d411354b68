// w4a8_math.cuh -- device helpers shared by the kernels: activation loads, the exact
// dequantise / SwiGLU epilogue arithmetic, the int8 mma.sync wrapper.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

namespace rkb200 {

template <bool HALF> struct ActType;
template <> struct ActType<true> { using type = uint16_t; };
template <> struct ActType<false> { using type = float; };

// 16 consecutive activations of one row as raw words (8 for binary16, 16 for fp32);
// elements at or beyond K read as zero.  `vec` says the row allows 16-byte loads.
template <bool HALF> struct Raw16 { uint32_t w[HALF ? 8 : 16]; };

// The element-by-element form (rows that do not allow 16-byte loads, the unit that straddles K) is kept out of line:
// the kernels are straight-line code executed once per launch, so every inlined copy of a rare path is instruction
// fetch on the critical path.
// (returns four words at a time: a vector return value stays in registers, a reference to the caller's unit would
// force that unit into local memory)
template <bool HALF>
__device__ __noinline__ uint4 load_words_ragged(const typename ActType<HALF>::type* row, int k0, int K)
{
    uint32_t w[4];
    if constexpr (HALF) {
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = (k0 + 2 * i < K) ? row[k0 + 2 * i] : 0u;
            const uint32_t hi = (k0 + 2 * i + 1 < K) ? row[k0 + 2 * i + 1] : 0u;
            w[i] = lo | (hi << 16);
        }
    } else {
        for (int i = 0; i < 4; ++i) w[i] = (k0 + i < K) ? __float_as_uint(row[k0 + i]) : 0u;
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <bool HALF>
__device__ __forceinline__ void load_raw(const typename ActType<HALF>::type* row, int k0, int K, bool vec, Raw16<HALF>& r)
{
    if (vec && k0 + 16 <= K) {
        if constexpr (HALF) {
            const uint4 a = *reinterpret_cast<const uint4*>(row + k0);
            const uint4 b = *reinterpret_cast<const uint4*>(row + k0 + 8);
            r.w[0] = a.x; r.w[1] = a.y; r.w[2] = a.z; r.w[3] = a.w;
            r.w[4] = b.x; r.w[5] = b.y; r.w[6] = b.z; r.w[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 f = *reinterpret_cast<const uint4*>(row + k0 + 4 * i);
                r.w[4 * i] = f.x; r.w[4 * i + 1] = f.y; r.w[4 * i + 2] = f.z; r.w[4 * i + 3] = f.w;
            }
        }
    } else {
        constexpr int per = HALF ? 8 : 4;      // elements per four words
#pragma unroll
        for (int i = 0; i < (HALF ? 2 : 4); ++i) {
            const uint4 f = load_words_ragged<HALF>(row, k0 + per * i, K);
            r.w[4 * i] = f.x; r.w[4 * i + 1] = f.y; r.w[4 * i + 2] = f.z; r.w[4 * i + 3] = f.w;
        }
    }
}
// max over the 16 magnitudes, as bit patterns (binary16: 15 bits, fp32: 31 bits)
template <bool HALF>
__device__ __forceinline__ uint32_t raw_maxbits(const Raw16<HALF>& r)
{
    uint32_t m = 0;
    if constexpr (HALF) {
#pragma unroll
        for (int i = 0; i < 8; ++i) m = max(m, max(r.w[i] & 0x7fffu, (r.w[i] >> 16) & 0x7fffu));
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) m = max(m, r.w[i] & 0x7fffffffu);
    }
    return m;
}
template <bool HALF>
__device__ __forceinline__ void raw_to_float(const Raw16<HALF>& r, float (&v)[16])
{
    if constexpr (HALF) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = __half2float(__ushort_as_half((uint16_t)(r.w[i] & 0xffffu)));
            v[2 * i + 1] = __half2float(__ushort_as_half((uint16_t)(r.w[i] >> 16)));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r.w[i]);
    }
}
template <bool HALF>
__device__ __forceinline__ void load16(const typename ActType<HALF>::type* row, int k0, int K, bool vec, float (&v)[16],
                                       uint32_t& maxbits)
{
    Raw16<HALF> r;
    load_raw<HALF>(row, k0, K, vec, r);
    maxbits = max(maxbits, raw_maxbits<HALF>(r));
    raw_to_float<HALF>(r, v);
}

// Degree-7 polynomial SiLU of the reference's production target, every rounding kept:
// src/rk_npu_swiglu_fp32_neon.h:17-41.
__device__ __forceinline__ float silu_poly(float g)
{
    float x = fminf(fmaxf(-g, -80.f), 80.f);
    const float n = floorf(fmaf(x, 1.4426950408889634f, 0.5f));
    float r = fmaf(-n, 0.693145751953125f, x);
    r = fmaf(-n, 1.428606765330187e-6f, r);
    float q = 1.f / 5040.f;
    q = fmaf(q, r, 1.f / 720.f);
    q = fmaf(q, r, 1.f / 120.f);
    q = fmaf(q, r, 1.f / 24.f);
    q = fmaf(q, r, 1.f / 6.f);
    q = fmaf(q, r, 0.5f);
    q = fmaf(q, r, 1.f);
    q = fmaf(q, r, 1.f);
    const float power = __int_as_float(((int)n + 127) << 23);
    const float d = __fadd_rn(1.f, __fmul_rn(q, power));
    return g < -80.f ? -0.f : __fdiv_rn(g, d);
}
// The same function for four arguments in lock step: every statement is applied to all four values before the next
// one.  Each value goes through exactly the operations of silu_poly (same bits); what changes is that the four
// dependent chains are interleaved in program order -- written one value after the other, sixteen evaluations took
// 2190 cycles per warp, in lock step 1420 (the divisions sit in separate basic blocks and are not interleaved by
// the compiler on its own).
__device__ __forceinline__ void silu_poly4(const float (&g)[4], float (&y)[4])
{
    float x[4], n[4], r[4], q[4], d[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = fminf(fmaxf(-g[j], -80.f), 80.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) n[j] = floorf(fmaf(x[j], 1.4426950408889634f, 0.5f));
#pragma unroll
    for (int j = 0; j < 4; ++j) r[j] = fmaf(-n[j], 0.693145751953125f, x[j]);
#pragma unroll
    for (int j = 0; j < 4; ++j) r[j] = fmaf(-n[j], 1.428606765330187e-6f, r[j]);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = fmaf(1.f / 5040.f, r[j], 1.f / 720.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = fmaf(q[j], r[j], 1.f / 120.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = fmaf(q[j], r[j], 1.f / 24.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = fmaf(q[j], r[j], 1.f / 6.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = fmaf(q[j], r[j], 0.5f);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = fmaf(q[j], r[j], 1.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = fmaf(q[j], r[j], 1.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) d[j] = __fadd_rn(1.f, __fmul_rn(q[j], __int_as_float(((int)n[j] + 127) << 23)));
#pragma unroll
    for (int j = 0; j < 4; ++j) y[j] = g[j] < -80.f ? -0.f : __fdiv_rn(g[j], d[j]);
}
__device__ __forceinline__ float dequant(int acc, float sx, float sw)
{
    return __fmul_rn(__fmul_rn(__int2float_rn(acc), sx), sw);
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// Four consecutive outputs of one token row: vector store when the address allows it.
__device__ __forceinline__ void store4_f32(float* out, const float (&y)[4], int valid)
{
    if (valid == 4 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) *reinterpret_cast<float4*>(out) = make_float4(y[0], y[1], y[2], y[3]);
    else for (int e = 0; e < valid; ++e) out[e] = y[e];
}
__device__ __forceinline__ void store4_f16(__half* out, const float (&y)[4], int valid)
{
    if (valid == 4 && (reinterpret_cast<uintptr_t>(out) & 7u) == 0) {
        const __half2 h0 = __halves2half2(__float2half_rn(y[0]), __float2half_rn(y[1]));
        const __half2 h1 = __halves2half2(__float2half_rn(y[2]), __float2half_rn(y[3]));
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&h0);
        pk.y = *reinterpret_cast<const uint32_t*>(&h1);
        *reinterpret_cast<uint2*>(out) = pk;
    } else for (int e = 0; e < valid; ++e) out[e] = __float2half_rn(y[e]);
}
__device__ __forceinline__ void store4_i32(int* out, const int (&v)[4], int valid)
{
    if (valid == 4 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) *reinterpret_cast<int4*>(out) = make_int4(v[0], v[1], v[2], v[3]);
    else for (int e = 0; e < valid; ++e) out[e] = v[e];
}
// Per-token scale from the magnitude bits of the row maximum:
// s = max(maximum / 127, FLT_MIN), 1 for a zero (or rejected) row; inverse = 1 / s.
__device__ __forceinline__ void scale_from_max(float maximum, bool bad, float& s, float& inv)
{
    s = (maximum == 0.f || bad) ? 1.0f : fmaxf(__fdiv_rn(maximum, 127.0f), FLT_MIN);
    inv = __frcp_rn(s);   // the correctly rounded reciprocal: the same value as the IEEE division 1 / s
}
// round half away from zero, then clamp to [-127, 127], without conversion instructions.
// |x| + 0.5 added with rounding TOWARD ZERO never reaches an integer the exact sum does not reach,
// so its floor is round-half-away of |x| (a round-to-nearest add would turn 0.49999997 + 0.5 into 1).
// A second toward-zero add of 1.5 * 2^23 leaves that floor in the low mantissa bits; the sign goes
// back on with two integer operations.
__device__ __forceinline__ int round_clamp(float x)
{
    const float s = fminf(__fadd_rz(fabsf(x), 0.5f), 127.0f);
    const int n = __float_as_int(__fadd_rz(s, 12582912.0f)) - 0x4B400000;   // floor(s): 0..127
    const int m = __float_as_int(x) >> 31;                                    // 0 or -1
    return (n ^ m) - m;
}
// Four products -> four int8 codes in one word (byte i = code of y[i]), ties away from zero.
// Magnitudes: |y| + 0.5 added toward zero, then 1.5 * 2^23 added toward zero leaves floor(|y| + 0.5) in the low byte of
// the float's bits (see round_clamp).  No clamp: every caller's scale is max(max|row| / 127, FLT_MIN) of the row the
// product comes from, so |y| <= 127 (1 + 2^-22) and the floor never exceeds 127.  Signs: one byte of ones per negative
// product (byte permutes that replicate the sign bit), then a bytewise two's-complement negation in five word
// operations: x = n ^ s; low seven bits of x plus one where s is set cannot carry out of their byte.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
    return d;
}
__device__ __forceinline__ uint32_t quantize4(float y0, float y1, float y2, float y3)
{
    const uint32_t g0 = __float_as_uint(__fadd_rz(__fadd_rz(fabsf(y0), 0.5f), 12582912.0f));
    const uint32_t g1 = __float_as_uint(__fadd_rz(__fadd_rz(fabsf(y1), 0.5f), 12582912.0f));
    const uint32_t g2 = __float_as_uint(__fadd_rz(__fadd_rz(fabsf(y2), 0.5f), 12582912.0f));
    const uint32_t g3 = __float_as_uint(__fadd_rz(__fadd_rz(fabsf(y3), 0.5f), 12582912.0f));
    const uint32_t n = prmt(prmt(g0, g1, 0x0040u), prmt(g2, g3, 0x0040u), 0x5410u);
    // selector nibbles 0xB / 0xF: byte 3 of the first / second operand with its sign bit replicated
    const uint32_t sgn = prmt(prmt(__float_as_uint(y0), __float_as_uint(y1), 0x00FBu), prmt(__float_as_uint(y2), __float_as_uint(y3), 0x00FBu), 0x5410u);
    const uint32_t x = n ^ sgn;
    return (((x & 0x7F7F7F7Fu) + (sgn & 0x01010101u)) ^ (x & 0x80808080u));
}
// the unit that straddles K: elements at or beyond K are zero codes (out of line; the values travel as vector arguments
// so that the caller's array stays in registers)
static __device__ __noinline__ uint4 quantize16_ragged(float4 a, float4 b, float4 c, float4 d, float inv, int k0, int K)
{
    const float v[16] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w, c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int q[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = (k0 + 4 * j + i < K) ? round_clamp(__fmul_rn(v[4 * j + i], inv)) : 0;
        w[j] = __byte_perm(__byte_perm((uint32_t)q[0], (uint32_t)q[1], 0x0040), __byte_perm((uint32_t)q[2], (uint32_t)q[3], 0x0040), 0x5410);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
// 16 activations -> 16 int8 codes packed in four words (ties away from zero; |code| <= 127 by the scale's construction).
__device__ __forceinline__ uint4 quantize16(const float (&v)[16], float inv, int k0, int K)
{
    if (k0 + 16 > K)
        return quantize16_ragged(make_float4(v[0], v[1], v[2], v[3]), make_float4(v[4], v[5], v[6], v[7]), make_float4(v[8], v[9], v[10], v[11]),
                                 make_float4(v[12], v[13], v[14], v[15]), inv, k0, K);
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        w[j] = quantize4(__fmul_rn(v[4 * j], inv), __fmul_rn(v[4 * j + 1], inv), __fmul_rn(v[4 * j + 2], inv), __fmul_rn(v[4 * j + 3], inv));
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// One 16-element unit from its raw words to int8 codes.  Out of line on purpose: a thread calls it up to three times
// (plus the tail loop), and four inlined copies of ~130 instructions are fetched once each on the critical path.
static __device__ __noinline__ uint4 quantize_words_half(uint4 lo, uint4 hi, float inv, int k0, int K)
{
    Raw16<true> raw;
    raw.w[0] = lo.x; raw.w[1] = lo.y; raw.w[2] = lo.z; raw.w[3] = lo.w;
    raw.w[4] = hi.x; raw.w[5] = hi.y; raw.w[6] = hi.z; raw.w[7] = hi.w;
    float v[16];
    raw_to_float<true>(raw, v);
    return quantize16(v, inv, k0, K);
}
static __device__ __noinline__ uint4 quantize_words_float(uint4 a, uint4 b, uint4 c, uint4 d, float inv, int k0, int K)
{
    const float v[16] = {__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w),
                         __uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z), __uint_as_float(b.w),
                         __uint_as_float(c.x), __uint_as_float(c.y), __uint_as_float(c.z), __uint_as_float(c.w),
                         __uint_as_float(d.x), __uint_as_float(d.y), __uint_as_float(d.z), __uint_as_float(d.w)};
    return quantize16(v, inv, k0, K);
}
// (the words travel as vector arguments, which the calling convention keeps in registers; a struct would go through
// the stack)
template <bool HALF>
__device__ __forceinline__ uint4 quantize_unit(const Raw16<HALF>& r, float inv, int k0, int K)
{
    if constexpr (HALF)
        return quantize_words_half(make_uint4(r.w[0], r.w[1], r.w[2], r.w[3]), make_uint4(r.w[4], r.w[5], r.w[6], r.w[7]), inv, k0, K);
    else
        return quantize_words_float(make_uint4(r.w[0], r.w[1], r.w[2], r.w[3]), make_uint4(r.w[4], r.w[5], r.w[6], r.w[7]),
                                    make_uint4(r.w[8], r.w[9], r.w[10], r.w[11]), make_uint4(r.w[12], r.w[13], r.w[14], r.w[15]), inv, k0, K);
}

} // namespace rkb200
