/*
 * w4a8_oracle.c -- CPU restatement of the reference W4A8 quantized-linear path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the parity tests,
 * the smoke test and the benchmark's CPU-baseline leg compare the CUDA library
 * against.  Nothing in the shipped library links, imports or calls it.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle_*.py)
 * against the known answers held by the reference's own tests and against the
 * reference's own CPU stages compiled from its sources (oracle/ref_glue.cpp),
 * on seeded inputs whose outputs are committed under tests/golden/.
 *
 * Each function cites the reference file:line it restates (paths are relative
 * to the reference project root).
 *
 * Plain C11, optional OpenMP for the integer contraction (the only O(M*K*N) part).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_OK 0
#define ORC_ERR_PARAM (-3) /* same value as RK_NPU_ERR_PARAM, include/rk_npu_common.h:30 */

/* ------------------------------------------------------------------ binary16
 * src/rk_npu_half_bits.h:8-27  (half -> float, exact, subnormals normalised,
 * NaN payload kept) and :28-53 (float -> half, round to nearest even, overflow
 * to infinity, values below half the smallest subnormal flush to signed zero). */
float orc_half_to_float(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 31u;
    uint32_t m = h & 1023u, bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {
            int shift = 0;
            while (!(m & 1024u)) { m <<= 1; ++shift; }
            bits = sign | (uint32_t)(127 - 14 - shift) << 23 | (m & 1023u) << 13;
        }
    } else if (e == 31) {
        bits = sign | 0x7f800000u | m << 13;
    } else {
        bits = sign | (e + 112u) << 23 | m << 13;
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t orc_float_to_half(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, biased = (x >> 23) & 255u;
    uint32_t man = x & 0x7fffffu;
    if (biased == 255u)
        return (uint16_t)(sign | 0x7c00u | (man ? ((man >> 13) | 0x200u) : 0u));
    const int e = (int)biased - 127 + 15;
    if (e >= 31)
        return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10)
            return (uint16_t)sign;
        man |= 0x800000u;
        const int shift = 14 - e;
        uint32_t hm = man >> shift;
        const uint32_t half_bit = 1u << (shift - 1);
        if ((man & half_bit) && ((man & (half_bit - 1)) || (hm & 1u)))
            ++hm;
        return (uint16_t)(sign | hm);
    }
    uint32_t h = sign | (uint32_t)e << 10 | man >> 13;
    if ((man & 0x1000u) && ((man & 0xfffu) || (h & 1u)))
        ++h; /* a carry out of the mantissa correctly bumps the exponent */
    return (uint16_t)h;
}

void orc_half_to_float_n(const uint16_t *src, float *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) dst[i] = orc_half_to_float(src[i]);
}
void orc_float_to_half_n(const float *src, uint16_t *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) dst[i] = orc_float_to_half(src[i]);
}

static inline float load_act(const void *A, int half, int64_t i)
{
    return half ? orc_half_to_float(((const uint16_t *)A)[i]) : ((const float *)A)[i];
}

/* --------------------------------------------------------- per-token scales
 * src/rk_npu_w4a8_quant.cpp:52-85 (scales_impl): full-row max|x|, any NaN/Inf
 * makes the call fail, s = max(maxabs/127, FLT_MIN) (1 for an all-zero row),
 * inverse = 1/s with an IEEE division. */
int orc_scales(const void *A, int half, int M, int K, float *scales, float *inverse)
{
    if (!A || M < 1 || K < 1 || !scales || !inverse) return ORC_ERR_PARAM;
    int bad = 0;
    for (int m = 0; m < M; ++m) {
        float maximum = 0.f;
        for (int k = 0; k < K; ++k) {
            const float x = load_act(A, half, (int64_t)m * K + k);
            if (!isfinite(x)) bad = 1;
            const float a = fabsf(x);
            if (a > maximum) maximum = a;
        }
        float s = 1.0f;
        if (maximum != 0.f) {
            s = maximum / 127.0f;
            if (s < FLT_MIN) s = FLT_MIN;
        }
        scales[m] = s;
        inverse[m] = 1.0f / s;
    }
    return bad ? ORC_ERR_PARAM : ORC_OK;
}

/* src/rk_npu_w4a8_quant.cpp:119-121: q = clamp(round_half_away(x * inverse), -127, 127).
 * The product is rounded to float before rounding to an integer (two steps). */
static inline int quant_code(float x, float inv)
{
    float r = roundf(x * inv);
    if (r > 127.f) r = 127.f;
    if (r < -127.f) r = -127.f;
    return (int)r;
}

void orc_quantize(const void *A, int half, int M, int K, const float *inverse, int8_t *q)
{
    for (int m = 0; m < M; ++m)
        for (int k = 0; k < K; ++k)
            q[(int64_t)m * K + k] = (int8_t)quant_code(load_act(A, half, (int64_t)m * K + k), inverse[m]);
}

/* src/rk_npu_w4a8_quant.cpp:122 : the reference splits each int8 code into two
 * signed int4 digits, high = q >> 4 and low = ((q & 15) ^ 8) read as a 4-bit
 * two's complement number, so that q = 16*high + low + 8.  Kept here only so
 * that tests can rebuild codes from the reference's packed buffers. */
void orc_msd_split(int8_t q, int *high, int *low)
{
    const uint8_t u = (uint8_t)q;
    const int h = u >> 4, l = (u & 15) ^ 8;
    *high = h >= 8 ? h - 16 : h;
    *low = l >= 8 ? l - 16 : l;
}

/* ------------------------------------------------------- integer contraction
 * tests/test_w4a8.cpp:31-37 : acc[m,n] = sum_k q[m,k] * B[k,n] in 64-bit, then
 * narrowed to int32 (the library's accumulator type, src/rk_npu_w4a8_output.cpp:70).
 * This equals correction + sum over waves of (16*hi + lo) whenever no INT16
 * partial saturates (src/rk_npu_w4a8_output.cpp:38-44, src/rk_npu_w4a8.cpp:236-242). */
void orc_gemm_i32(const int8_t *q, const int8_t *B, int M, int K, int N, int32_t *acc)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        int64_t *row = (int64_t *)calloc((size_t)N, sizeof(int64_t));
        for (int k = 0; k < K; ++k) {
            const int64_t a = q[(int64_t)m * K + k];
            if (!a) continue;
            const int8_t *b = B + (int64_t)k * N;
            for (int n = 0; n < N; ++n) row[n] += a * b[n];
        }
        for (int n = 0; n < N; ++n) acc[(int64_t)m * N + n] = (int32_t)row[n];
        free(row);
    }
}

/* Same contraction restricted to a list of columns (the reference's sampled
 * check: 17 evenly spaced columns, src/rk_npu_w4a8_tune_data.cpp:30-33). */
void orc_gemm_i32_columns(const int8_t *q, const int8_t *B, int M, int K, int N,
                          const int *columns, int count, int32_t *acc)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int c = 0; c < count; ++c) {
            const int n = columns[c];
            int64_t sum = 0;
            for (int k = 0; k < K; ++k)
                sum += (int64_t)q[(int64_t)m * K + k] * B[(int64_t)k * N + n];
            acc[(int64_t)m * count + c] = (int32_t)sum;
        }
}

/* ------------------------------------------------------------------ dequant
 * src/rk_npu_w4a8_output.cpp:226-262 (w4a8_dequant) and :70-76 (combine8):
 * y = (float(acc) * a_scale[m]) * w_scale[n], two roundings in that order, then
 * one round-to-nearest-even cast when the output is binary16. */
void orc_dequant(int M, int N, const int32_t *acc, const float *a_scale, const float *w_scale,
                 int half, void *out)
{
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            const float t = (float)acc[(int64_t)m * N + n] * a_scale[m];
            const float y = t * w_scale[n];
            if (half) ((uint16_t *)out)[(int64_t)m * N + n] = orc_float_to_half(y);
            else ((float *)out)[(int64_t)m * N + n] = y;
        }
}

/* ================================================================ typed W8A8 operators
 * include/rk_npu_quant_matmul.h:358-372, src/rk_npu_cpu_kernels.cpp (scalar branches).
 * Dynamic scale: max|x| / 127 when the maximum is positive, else 1 (:576-589, :853-871).  std::max(a, b) keeps a
 * when b is NaN, so a NaN never raises the maximum; no lower clamp, no rejection of non-finite input. */
void orc_w8_scales(const void *A, int half, int M, int K, float *scales)
{
    for (int m = 0; m < M; ++m) {
        float maximum = 0.f;
        for (int k = 0; k < K; ++k) {
            const float a = fabsf(load_act(A, half, (int64_t)m * K + k));
            if (maximum < a) maximum = a;
        }
        scales[m] = maximum > 0.f ? maximum / 127.0f : 1.0f;
    }
}

/* :126-131 (quantize_s8_symmetric) and :598-606: a scale that is not positive gives zeros; otherwise
 * q = max(-127, min(127, round(x * (1 / scale)))) with std::min / std::max argument order, so NaN -> 127. */
void orc_w8_quantize(const void *A, int half, int M, int K, const float *scales, int8_t *q)
{
    for (int m = 0; m < M; ++m) {
        const float scale = scales[m];
        for (int k = 0; k < K; ++k) {
            int8_t code = 0;
            if (scale > 0.0f) {
                float r = roundf(load_act(A, half, (int64_t)m * K + k) * (1.0f / scale));
                r = (r < 127.0f) ? r : 127.0f;         /* std::min(127.0f, r) */
                r = (-127.0f < r) ? r : -127.0f;       /* std::max(-127.0f, r) */
                code = (int8_t)r;
            }
            q[(int64_t)m * K + k] = code;
        }
    }
}

/* One W8A8 linear: scales (dynamic, or the caller's when a_scale_static is given), codes, exact int32 sums modulo 2^32
 * (include/rk_npu_quant_matmul.h:335-340), y = float(acc) * a_scale[m] * w_scale[n] evaluated left to right
 * (src/rk_npu_cpu_kernels.cpp:1312), one more rounding for binary16 output. */
int orc_w8_linear(const void *A, int half, int M, int K, int N, const int8_t *B, const float *w_scale,
                  const float *a_scale_static, void *out, int32_t *acc, float *scales_used, int8_t *codes)
{
    if (!A || !B || !w_scale || !out || !acc || !scales_used || !codes || M < 1 || K < 1 || N < 1) return ORC_ERR_PARAM;
    if (a_scale_static) memcpy(scales_used, a_scale_static, sizeof(float) * (size_t)M);
    else orc_w8_scales(A, half, M, K, scales_used);
    orc_w8_quantize(A, half, M, K, scales_used, codes);
    orc_gemm_i32(codes, B, M, K, N, acc);
    orc_dequant(M, N, acc, scales_used, w_scale, half, out);
    return ORC_OK;
}

/* ------------------------------------------------------------------- SwiGLU
 * Two activations exist in the reference:
 *   mode 0: src/rk_npu_w4a8_swiglu.cpp:71  y = (g / (1 + expf(-g))) * u
 *           (what the reference computes when built for a non-ARM host);
 *   mode 1: src/rk_npu_swiglu_fp32_neon.h:13-51, the degree-7 polynomial the
 *           reference uses on its production target: the argument -g is clamped
 *           to [-80, 80], n = floor(x*log2(e) + 0.5) with one fused multiply-add,
 *           two fused subtractions of n*ln2 (hi, lo), Horner with fused steps from
 *           1/5040 down to 1, 2^n rebuilt from exponent bits, the denominator
 *           1 + p*2^n as a separate multiply then add, an IEEE division, and
 *           g < -80 mapped to -0.  Restated here with fmaf so every rounding is
 *           the same as the vector code's. */
float orc_silu_expf(float g) { return g / (1.f + expf(-g)); }

float orc_silu_poly(float g)
{
    float x = -g;
    if (x > 80.f) x = 80.f;
    if (x < -80.f) x = -80.f;
    const float n = floorf(fmaf(x, 1.4426950408889634f, 0.5f));
    float r = fmaf(-n, 0.693145751953125f, x);
    r = fmaf(-n, 1.428606765330187e-6f, r);
    float p = 1.f / 5040.f;
    p = fmaf(p, r, 1.f / 720.f);
    p = fmaf(p, r, 1.f / 120.f);
    p = fmaf(p, r, 1.f / 24.f);
    p = fmaf(p, r, 1.f / 6.f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.f);
    p = fmaf(p, r, 1.f);
    const int32_t e = ((int32_t)n + 127) << 23;
    float power;
    memcpy(&power, &e, 4);
    volatile float scaled = p * power; /* separate multiply: no contraction into the add */
    const float d = 1.f + scaled;
    return g < -80.f ? -0.f : g / d;
}

/* src/rk_npu_w4a8_swiglu.cpp:12-91 (finish_swiglu): the accumulator holds
 * [gate(F), up(F)] columns; both are dequantised exactly as in orc_dequant, the
 * activation is applied to gate, multiplied by up, stored as compact [M,F] fp32;
 * row_max_bits[m] = max over the row of (bits(y) & 0x7fffffff) when requested. */
void orc_swiglu(int M, int F, const int32_t *acc, const float *a_scale, const float *w_scale,
                int mode, float *middle, uint32_t *row_max_bits)
{
    const int N = 2 * F;
    for (int m = 0; m < M; ++m) {
        uint32_t maximum = 0;
        for (int f = 0; f < F; ++f) {
            const float g = ((float)acc[(int64_t)m * N + f] * a_scale[m]) * w_scale[f];
            const float u = ((float)acc[(int64_t)m * N + F + f] * a_scale[m]) * w_scale[F + f];
            const float s = mode ? orc_silu_poly(g) : orc_silu_expf(g);
            volatile float y = s * u;
            middle[(int64_t)m * F + f] = y;
            uint32_t bits;
            float yy = y;
            memcpy(&bits, &yy, 4);
            bits &= 0x7fffffffu;
            if (bits > maximum) maximum = bits;
        }
        if (row_max_bits) row_max_bits[m] = maximum;
    }
}

/* src/rk_npu_w4a8_quant.cpp:145-161 (w4a8_finish_scales): turn the collected
 * magnitude bit patterns into scales; any pattern >= +inf (0x7f800000) fails. */
int orc_finish_scales(int M, const uint32_t *row_max_bits, float *scales, float *inverse)
{
    for (int m = 0; m < M; ++m) {
        const uint32_t bits = row_max_bits[m];
        if (bits >= 0x7f800000u) return ORC_ERR_PARAM;
        float maximum;
        memcpy(&maximum, &bits, 4);
        float s = 1.f;
        if (maximum != 0.f) {
            s = maximum / 127.f;
            if (s < FLT_MIN) s = FLT_MIN;
        }
        scales[m] = s;
        inverse[m] = 1.f / s;
    }
    return ORC_OK;
}

/* ------------------------------------------------------------ complete calls
 * src/rk_npu_w4a8.cpp:98-151 (run_locked) for one linear: scan, quantise, contract,
 * dequantise.  acc_out (optional) receives the int32 accumulators. */
int orc_linear(const void *A, int half, int M, int K, int N, const int8_t *B, const float *w_scale,
               void *out, int32_t *acc_out, float *scales_out)
{
    float *s = (float *)malloc(sizeof(float) * (size_t)M * 2);
    int8_t *q = (int8_t *)malloc((size_t)M * K);
    int32_t *acc = acc_out ? acc_out : (int32_t *)malloc(sizeof(int32_t) * (size_t)M * N);
    int rc = orc_scales(A, half, M, K, s, s + M);
    if (!rc) {
        orc_quantize(A, half, M, K, s + M, q);
        orc_gemm_i32(q, B, M, K, N, acc);
        orc_dequant(M, N, acc, s, w_scale, half, out);
        if (scales_out) memcpy(scales_out, s, sizeof(float) * (size_t)M);
    }
    if (!acc_out) free(acc);
    free(q);
    free(s);
    return rc;
}

/* src/rk_npu_w4a8.cpp:354-380 (rk_npu_w4a8_run_ffn_f32): gate/up projection with the
 * fused SwiGLU epilogue collecting row maxima, scales finished from those maxima
 * (no rescan), down projection quantising `middle` with the reused scales.
 * Returns ORC_ERR_PARAM for non-finite input or non-finite middle (in which case
 * the down projection is not evaluated). Optional outputs may be NULL. */
int orc_ffn(const float *A, int M, int K, int F, int N, const int8_t *B_gate_up,
            const float *scale_gate_up, const int8_t *B_down, const float *scale_down, int mode,
            float *middle, float *C, int32_t *acc_gate_up, int32_t *acc_down, float *scales_down_in)
{
    const int N2 = 2 * F;
    float *s = (float *)malloc(sizeof(float) * (size_t)M * 4);
    uint32_t *maxima = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)M);
    int8_t *q = (int8_t *)malloc((size_t)M * (K > F ? K : F));
    int32_t *acc1 = acc_gate_up ? acc_gate_up : (int32_t *)malloc(sizeof(int32_t) * (size_t)M * N2);
    int32_t *acc2 = acc_down ? acc_down : (int32_t *)malloc(sizeof(int32_t) * (size_t)M * N);
    int rc = orc_scales(A, 0, M, K, s, s + M);
    if (!rc) {
        orc_quantize(A, 0, M, K, s + M, q);
        orc_gemm_i32(q, B_gate_up, M, K, N2, acc1);
        orc_swiglu(M, F, acc1, s, scale_gate_up, mode, middle, maxima);
        rc = orc_finish_scales(M, maxima, s + 2 * M, s + 3 * M);
    }
    if (!rc) {
        orc_quantize(middle, 0, M, F, s + 3 * M, q);
        orc_gemm_i32(q, B_down, M, F, N, acc2);
        orc_dequant(M, N, acc2, s + 2 * M, scale_down, 0, C);
        if (scales_down_in) memcpy(scales_down_in, s + 2 * M, sizeof(float) * (size_t)M);
    }
    if (!acc_down) free(acc2);
    if (!acc_gate_up) free(acc1);
    free(q);
    free(maxima);
    free(s);
    return rc;
}

/* -------------------------------------------------------------- weight side
 * src/rk_npu_w4a8.cpp:229-242: scales must be finite and > 0; codes must lie in
 * [-8, 7]; correction[n] = 8 * sum_k B[k,n]. Returns ORC_ERR_PARAM otherwise. */
int orc_weight_check(int K, int N, const int8_t *B, const float *w_scale, int32_t *correction)
{
    for (int n = 0; n < N; ++n) {
        if (!isfinite(w_scale[n]) || !(w_scale[n] > 0)) return ORC_ERR_PARAM;
        if (correction) correction[n] = 0;
    }
    for (int k = 0; k < K; ++k)
        for (int n = 0; n < N; ++n) {
            const int v = B[(int64_t)k * N + n];
            if (v < -8 || v > 7) return ORC_ERR_PARAM;
            if (correction) correction[n] += 8 * v;
        }
    return ORC_OK;
}

/* src/rk_npu_i4_bounds.cpp:9-69 (bound_i4_weights).  For a fixed partition of K
 * into tiles of t*32 elements, a column is safe when, inside every tile,
 *   P = sum(w >= 0 ? 7*w : -8*w) <= 32767  and  Q = sum(w >= 0 ? 8*w : -7*w) <= 32768,
 * i.e. no int4 x int4 partial can leave INT16.  requested == 0 examines every
 * t in 1..min(64, ceil(K/32)); a positive request examines that tile (and the
 * optional smaller fallback) only.  Outputs: the largest safe tile, the maxima
 * of P and Q seen for it, and a bit mask with bit (t-1) set for every safe t.
 * Columns are walked in slabs of 128 and a tile stops being examined (and its
 * maxima stop growing) at the first unsafe column, exactly as the reference. */
int orc_bound_i4_weights(int K, int N, const int8_t *B, int requested, int fallback,
                         int *k_tile, int64_t *positive, int64_t *negative, uint64_t *safe_tiles)
{
    if (!B || K < 1 || K > INT32_MAX / 64 || N < 1 || N > INT32_MAX - 63 || requested < 0 ||
        requested > 2048 || requested % 32 || fallback < 0 || fallback % 32 ||
        (fallback && fallback >= requested))
        return ORC_ERR_PARAM;
    const int blocks = (K + 31) / 32;
    const int limit = requested ? requested / 32 : (blocks < 64 ? blocks : 64);
    int safe[65] = {0};
    int64_t max_pos[65] = {0}, max_neg[65] = {0};
    for (int t = 1; t <= limit; ++t) safe[t] = !requested || t == limit || t * 32 == fallback;
    const int slab = 128;
    int64_t *pos = (int64_t *)malloc(sizeof(int64_t) * (size_t)(blocks + 1) * slab * 2);
    int64_t *neg = pos + (size_t)(blocks + 1) * slab;
    for (int n0 = 0; n0 < N; n0 += slab) {
        const int width = N - n0 < slab ? N - n0 : slab;
        memset(pos, 0, sizeof(int64_t) * (size_t)width);
        memset(neg, 0, sizeof(int64_t) * (size_t)width);
        for (int b = 0; b < blocks; ++b) {
            int64_t *p = pos + (size_t)(b + 1) * width, *q = neg + (size_t)(b + 1) * width;
            memcpy(p, p - width, sizeof(int64_t) * (size_t)width);
            memcpy(q, q - width, sizeof(int64_t) * (size_t)width);
            const int kend = (b + 1) * 32 < K ? (b + 1) * 32 : K;
            for (int k = b * 32; k < kend; ++k) {
                const int8_t *row = B + (int64_t)k * N + n0;
                for (int n = 0; n < width; ++n) {
                    const int w = row[n];
                    if (w < -8 || w > 7) { free(pos); return ORC_ERR_PARAM; }
                    p[n] += w >= 0 ? 7 * w : -8 * w;
                    q[n] += w >= 0 ? 8 * w : -7 * w;
                }
            }
        }
        for (int t = 1; t <= limit; ++t) {
            if (!safe[t]) continue;
            for (int b = 0; b < blocks && safe[t]; b += t) {
                const int e = b + t < blocks ? b + t : blocks;
                for (int n = 0; n < width; ++n) {
                    const int64_t hi = pos[(size_t)e * width + n] - pos[(size_t)b * width + n];
                    const int64_t lo = neg[(size_t)e * width + n] - neg[(size_t)b * width + n];
                    if (hi > max_pos[t]) max_pos[t] = hi;
                    if (lo > max_neg[t]) max_neg[t] = lo;
                    if (hi > 32767 || lo > 32768) { safe[t] = 0; break; }
                }
            }
        }
    }
    free(pos);
    uint64_t mask = 0;
    for (int t = 1; t <= limit; ++t)
        if (safe[t]) mask |= (uint64_t)1 << (t - 1);
    for (int t = limit; t >= 1; --t)
        if (safe[t]) {
            *k_tile = t * 32;
            *positive = max_pos[t];
            *negative = max_neg[t];
            *safe_tiles = mask;
            return ORC_OK;
        }
    return ORC_ERR_PARAM;
}

/* src/rk_npu_autotune_common.cpp:83-89 (tune::Hash): 64-bit FNV-1a; integers are
 * mixed as eight little-endian bytes.  src/rk_npu_w4a8.cpp:275-277: the weight
 * fingerprint hashes K, N, the K*N code bytes and the N fp32 scales. */
uint64_t orc_fnv_bytes(uint64_t h, const void *p, size_t n)
{
    const uint8_t *b = (const uint8_t *)p;
    for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 1099511628211ull; }
    return h;
}
uint64_t orc_fnv_mix(uint64_t h, uint64_t v)
{
    for (int i = 0; i < 8; ++i) { const uint8_t b = (uint8_t)(v >> (8 * i)); h = orc_fnv_bytes(h, &b, 1); }
    return h;
}
uint64_t orc_weight_fingerprint(int K, int N, const int8_t *B, const float *w_scale)
{
    uint64_t h = 1469598103934665603ull;
    h = orc_fnv_mix(h, (uint64_t)(int64_t)K);
    h = orc_fnv_mix(h, (uint64_t)(int64_t)N);
    h = orc_fnv_bytes(h, B, (size_t)K * N);
    h = orc_fnv_bytes(h, w_scale, (size_t)N * sizeof(float));
    return h;
}

/* ------------------------------------------------------------------ routed experts (rk_npu_moe_w8.h)
 *
 * The routed operator quantises with round-to-nearest-EVEN and without a lower clamp on the scale, unlike the
 * dense W4A8 path (src/rk_npu_moe_cpu.cpp:21-24 "MoE retains nearest-even rounding", :80 "scale=1 for all-zero
 * rows").  Pinned against the reference's compiled swiglu_quantize_row (its x86 form evaluates the sigmoid with
 * std::exp: mode 0 here); mode 1 is the degree-7 polynomial its production target shares with the dense path. */

/* src/rk_npu_moe_w8.cpp:317-343 (quantize<ValidateInput>): maximum of |x|, scale = max ? max/127 : 1,
 * inverse = 1/scale, code = nearest-even(clamp(x*inverse, -127, 127)).  With `validate` a non-finite element, a
 * scale that is not positive or an infinite inverse rejects the row (return 1). */
int orc_moe_quantize_row(const float *x, int n, int validate, int8_t *q, float *scale_out)
{
    float maximum = 0.f;
    for (int i = 0; i < n; ++i) {
        if (validate && !isfinite(x[i])) return 1;
        const float a = fabsf(x[i]);
        if (a > maximum) maximum = a;
    }
    const float scale = maximum != 0.f ? maximum / 127.f : 1.f;
    const float inverse = 1.f / scale;
    if (validate && (!(scale > 0.f) || !isfinite(inverse))) return 1;
    for (int i = 0; i < n; ++i) {
        float v = x[i] * inverse;
        if (v > 127.f) v = 127.f;
        if (v < -127.f) v = -127.f;
        q[i] = (int8_t)lrintf(v);   /* default rounding mode: to nearest, ties to even */
    }
    *scale_out = scale;
    return 0;
}

/* src/rk_npu_moe_cpu.cpp:47-115 (swiglu_quantize_row), plain int8 output: acc holds the row's [gate(I), up(I)]
 * int32 sums; both are dequantised as (float(sum) * input_scale) * weight_scale, y = silu(gate) * up, the row
 * maximum is taken on the bit patterns, and the row is re-quantised with the rule above.  Returns the scale. */
float orc_moe_middle_row(const int32_t *acc, int I, float input_scale, const float *w_scale, int mode, int8_t *q)
{
    float hidden[512];
    uint32_t maximum = 0;
    for (int n = 0; n < I; ++n) {
        const float g = ((float)acc[n] * input_scale) * w_scale[n];
        const float u = ((float)acc[I + n] * input_scale) * w_scale[I + n];
        const float s = mode ? orc_silu_poly(g) : orc_silu_expf(g);
        volatile float y = s * u;
        hidden[n] = y;
        float yy = y;
        uint32_t bits;
        memcpy(&bits, &yy, 4);
        bits &= 0x7fffffffu;
        if (bits > maximum) maximum = bits;
    }
    float maxabs;
    memcpy(&maxabs, &maximum, 4);
    const float scale = maximum ? maxabs / 127.f : 1.f;
    const float inverse = 1.f / scale;
    for (int n = 0; n < I; ++n) {
        float v = hidden[n] * inverse;
        if (v > 127.f) v = 127.f;
        if (v < -127.f) v = -127.f;
        q[n] = (int8_t)lrintf(v);
    }
    return scale;
}

/* The whole operator for int8 experts: src/rk_npu_moe_w8.cpp:570-817 (Workspace::run) and the independent
 * reference of tests/test_moe_w8.cpp:27-46.  Experts are flat arrays, expert e at e * stride:
 * gate_up [E][H][2I], gate_up_scales [E][2I], down [E][I][H], down_scales [E][H]; E = routed + shared, the
 * shared expert last.  A route with coefficient 0 is left out; the shared expert counts with coefficient 1;
 * the sum over a token's slots runs in slot order with one fused multiply-add per term (the production
 * target's vfmaq).  Validation as in the original: ids in range, coefficients finite and >= 0, row scales
 * finite and > 0.  Returns 0, or 1 for rejected arguments (out untouched). */
int orc_moe_run(int rows, int H, int I, int routed, int shared, int top, const int8_t *gate_up,
                const float *gate_up_scales, const int8_t *down, const float *down_scales, const int8_t *input,
                const float *row_scales, const int32_t *ids, const float *routes, int mode, float *out)
{
    for (int i = 0; i < rows * top; ++i)
        if (ids[i] < 0 || ids[i] >= routed || !isfinite(routes[i]) || routes[i] < 0.f) return 1;
    for (int r = 0; r < rows; ++r)
        if (!(row_scales[r] > 0.f) || !isfinite(row_scales[r])) return 1;
    int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * 2 * (size_t)I);
    int8_t *q = (int8_t *)malloc((size_t)I);
    float *sum = (float *)malloc(sizeof(float) * (size_t)H);
    if (!acc || !q || !sum) { free(acc); free(q); free(sum); return 2; }
    for (int r = 0; r < rows; ++r) {
        for (int n = 0; n < H; ++n) sum[n] = 0.f;
        for (int slot = 0; slot < top + shared; ++slot) {
            const float coefficient = slot < top ? routes[r * top + slot] : 1.f;
            if (slot < top && coefficient == 0.f) continue;
            const int e = slot < top ? ids[r * top + slot] : routed;
            const int8_t *G = gate_up + (size_t)e * H * 2 * I;
            const int8_t *D = down + (size_t)e * I * H;
            for (int c = 0; c < 2 * I; ++c) {
                int32_t a = 0;
                for (int k = 0; k < H; ++k) a += (int32_t)input[(size_t)r * H + k] * (int32_t)G[(size_t)k * 2 * I + c];
                acc[c] = a;
            }
            const float scale = orc_moe_middle_row(acc, I, row_scales[r], gate_up_scales + (size_t)e * 2 * I, mode, q);
            for (int n = 0; n < H; ++n) {
                int32_t a = 0;
                for (int k = 0; k < I; ++k) a += (int32_t)q[k] * (int32_t)D[(size_t)k * H + n];
                const float value = ((float)a * scale) * down_scales[(size_t)e * H + n];
                sum[n] = fmaf(value, coefficient, sum[n]);
            }
        }
        memcpy(out + (size_t)r * H, sum, sizeof(float) * (size_t)H);
    }
    free(acc); free(q); free(sum);
    return 0;
}

/* ---------------------------------------------------------------- residual add + RMSNorm (rk_npu_add_rmsnorm_f16.h)
 * The original runs this on its NPU only; what its result must equal is stated by its board test
 * (tests/test_add_rmsnorm_f16.cpp:96-113), restated here on row-major [M, D] fp16 bit patterns:
 *   sum  = fp16(float(x) + float(residual))                       (must match bit for bit, :104,107-108)
 *   inv  = 1 / sqrt(sum over d of double(sum)^2 / D + eps)        (:105-106,110; the squares are added in order of d)
 *   norm = fp16(float(double(sum) * inv * double(gamma)))         (:112-113; the device is allowed 0.04 around it)
 */
void orc_add_rmsnorm_f16(int M, int D, float eps, const uint16_t *x, const uint16_t *residual, const uint16_t *gamma,
                         uint16_t *residual_out, uint16_t *norm_out)
{
    for (int m = 0; m < M; ++m) {
        const size_t row = (size_t)m * D;
        double variance = 0.0;
        for (int d = 0; d < D; ++d) {
            residual_out[row + d] = orc_float_to_half(orc_half_to_float(x[row + d]) + orc_half_to_float(residual[row + d]));
            const double v = orc_half_to_float(residual_out[row + d]);
            variance += v * v;
        }
        const double inv = 1.0 / sqrt(variance / D + eps);
        for (int d = 0; d < D; ++d)
            norm_out[row + d] = orc_float_to_half((float)(orc_half_to_float(residual_out[row + d]) * inv * orc_half_to_float(gamma[d])));
    }
}
