// ref_glue.cpp -- drives the REFERENCE's own CPU w4a8 stages, compiled from the
// reference sources where they lie (see oracle/Makefile), so that the C
// restatement in w4a8_oracle.c can be validated against them and so that the
// benchmark can time the reference's CPU path on the host cores.
//
// TEST INFRASTRUCTURE ONLY: nothing in the shipped library links this file.
//
// The reference executes the int4 x int4 -> int16 contraction on an RK3588 NPU
// and ships no software model of it.  `npu_standin` below restates that single
// step on the CPU in the reference's native buffer layouts
// (src/rk_npu_i4_regs.h:11-16: A[K/32, rows, 32], B[N/64, K/32, 64, 32],
// C[N/8, rows, 8] INT16; index formulas as asserted by
// tests/test_w4a8_reduction.cpp:56-68 and tests/test_i4_cpu.cpp:24,34).
// Everything else -- scales, quantise + MSD split + packing, weight packing,
// tile plan, split-K reconstruction, dequantisation, fused SwiGLU, row maxima,
// scale finishing -- is the reference's compiled code.
#include "rk_npu_w4a8_cpu.h"
#include "rk_npu_i4_cpu.h"
#include "rk_npu_i4_bounds.h"
#include "rk_npu_w4a8_tune_internal.h"
#include "rk_npu_half_bits.h"
#include "rk_npu_cpu_kernels.h"
#include "rk_npu_quant_matmul.h"
#include "rk_npu_moe_cpu.h"
#include <algorithm>
#include <chrono>
#include <cstring>
#include <vector>
#include <omp.h>

using namespace rknpu2_matmul_open::detail;

namespace {
using Clock = std::chrono::steady_clock;
double since(Clock::time_point t) { return std::chrono::duration<double, std::micro>(Clock::now() - t).count(); }
inline int align_to(int x, int a) { return (x + a - 1) / a * a; }
inline int nibble(uint8_t byte, int j) { const int v = (j & 1) ? (byte & 15) : (byte >> 4); return v >= 8 ? v - 16 : v; }

struct Layer {
    int K = 0, N = 0, k_tile = 0;
    std::vector<uint8_t> packed;   // all waves, reference B layout
    std::vector<int32_t> correction;
    std::vector<float> scales;
};

int prepare_layer(Layer& L, int K, int N, int k_tile, const int8_t* B, const float* w_scale) {
    L.K = K; L.N = N; L.k_tile = k_tile;
    const int pn = align_to(N, 64);
    L.packed.assign(size_t(align_to(K, 32)) * pn / 2 + size_t((K + k_tile - 1) / k_tile) * 16 * pn, 0);
    size_t offset = 0;
    for (int k0 = 0; k0 < K;) {
        const int k = std::min(k_tile, K - k0), pk = align_to(k, 32);
        const int rc = pack_i4_weights(K, N, k0, k, pk, pn, B, L.packed.data() + offset);
        if (rc) return rc;
        offset += size_t(pk) * pn / 2;
        k0 += k;
    }
    L.scales.assign(w_scale, w_scale + N);
    L.correction.assign(N, 0);
    for (int k = 0; k < K; ++k)
        for (int n = 0; n < N; ++n) L.correction[n] += 8 * B[size_t(k) * N + n];   // src/rk_npu_w4a8.cpp:236-242
    return RK_NPU_OK;
}

// One K wave of the NPU step for every tile of the plan. Returns saturated count.
int64_t npu_standin(const std::vector<I4Tile>& tiles, int pk, const uint8_t* a_wave,
                    const uint8_t* b_wave, int16_t* partial) {
    int64_t saturated = 0;
    const int kb_count = pk / 32;
    for (const auto& t : tiles) {
        const uint8_t* a_panel = a_wave + size_t(t.m0) * pk / 2;
        std::vector<int8_t> a(size_t(t.m) * pk);
        for (int r = 0; r < t.m; ++r)
            for (int j = 0; j < pk; ++j)
                a[size_t(r) * pk + j] = int8_t(nibble(a_panel[(size_t(j / 32) * t.m + r) * 16 + (j % 32) / 2], j));
        int16_t* out = partial + t.output_offset / 2;
#pragma omp parallel for schedule(static) reduction(+ : saturated)
        for (int n = 0; n < t.n; ++n) {
            const int gn = t.n0 + n;
            std::vector<int8_t> b(pk);
            for (int kb = 0; kb < kb_count; ++kb) {
                const uint8_t* row = b_wave + ((size_t(gn / 64) * kb_count + kb) * 64 + gn % 64) * 16;
                for (int j = 0; j < 32; ++j) b[kb * 32 + j] = int8_t(nibble(row[j / 2], j));
            }
            for (int r = 0; r < t.m; ++r) {
                int32_t sum = 0;
                const int8_t* ar = a.data() + size_t(r) * pk;
                for (int j = 0; j < pk; ++j) sum += int(ar[j]) * int(b[j]);
                if (sum > 32767) { sum = 32767; ++saturated; }
                if (sum < -32768) { sum = -32768; ++saturated; }
                out[(size_t(n / 8) * t.m + r) * 8 + n % 8] = int16_t(sum);
            }
        }
    }
    return saturated;
}

struct Geometry { int m_tile, n_tile; uint32_t mask; int threads; };

// One projection through the reference stages. scale_source != nullptr reuses
// scales (the FFN's down projection, src/rk_npu_w4a8.cpp:112-121,376).
int run_projection(const Layer& L, const Geometry& g, const void* A, bool half, int M, void* out,
                   bool swiglu, uint32_t* row_maxima, float* scales, float* inverse,
                   bool reuse_scales, int32_t* acc_out, int64_t* saturated, double* stage_us) {
    const int K = L.K, N = L.N, kt = L.k_tile, pn = align_to(N, 64);
    rk_npu_i4_config cfg{M * 2, N, K, g.m_tile * 2, kt, g.n_tile, g.mask, 500, 0, g.threads};
    uint32_t starts[3]{}, counts[3]{};
    const auto tiles = i4_tiles(cfg, starts, counts, I4InputLayout::Native);
    auto t0 = Clock::now();
    int rc = RK_NPU_OK;
    if (!reuse_scales) rc = w4a8_scales(A, half, M, K, g.threads, scales, inverse);
    if (stage_us) stage_us[0] += since(t0);
    if (rc) return rc;
    W4A8Input input{A, half, M, K, scales, inverse, g.threads, I4InputLayout::Native};
    std::vector<int32_t> accumulator(size_t(M) * pn);
    std::vector<W4A8SwiGLUPair> pairs;
    if (swiglu) pairs = w4a8_swiglu_pairs(N, tiles);
    W4A8Reduction reduction{accumulator.data(), L.correction.data(), scales, L.scales.data(), out, half,
                            swiglu ? &pairs : nullptr, row_maxima, M + 16};
    const int waves = (K + kt - 1) / kt;
    std::vector<uint8_t> a_wave(size_t(M) * 2 * align_to(std::min(K, kt), 32) / 2 + 64);
    std::vector<int16_t> partial(size_t(M) * 2 * pn + 64);
    size_t weight_offset = 0;
    for (int w = 0; w < waves && !rc; ++w) {
        const int k0 = w * kt, k = std::min(kt, K - k0), pk = align_to(k, 32);
        t0 = Clock::now();
        std::memset(a_wave.data(), 0, size_t(M) * 2 * pk / 2);
        for (int m0 = 0; m0 < cfg.M && !rc;) {   // src/rk_npu_i4_plan.cpp:218-226
            const int rows = i4_m_rows(cfg.M - m0, cfg.m_tile, I4InputLayout::Native);
            rk_npu_i4_input_tile tile{m0, rows, k0, k, pk, a_wave.data() + size_t(m0) * pk / 2, uint64_t(rows) * pk / 2};
            rc = w4a8_pack(&input, &tile);
            m0 += rows;
        }
        if (stage_us) stage_us[1] += since(t0);
        if (rc) break;
        t0 = Clock::now();
        const int64_t sat = npu_standin(tiles, pk, a_wave.data(), L.packed.data() + weight_offset, partial.data());
        if (saturated) *saturated += sat;
        if (stage_us) stage_us[2] += since(t0);
        t0 = Clock::now();
        rc = w4a8_reduce_tiles(reduction, cfg, tiles, w, waves, partial.data());
        if (stage_us) stage_us[3] += since(t0);
        weight_offset += size_t(pk) * pn / 2;
    }
    if (!rc && acc_out && waves > 1 && !swiglu) {
        // The final wave writes C directly; rebuild the int32 the epilogue saw:
        // accumulator (waves 0..n-2) + last partial (native layout -> row major).
        for (const auto& t : tiles)
            for (int r = 0; r < t.m / 2; ++r)
                for (int n = 0; n < t.logical_n; ++n) {
                    const size_t index = (size_t(n / 8) * (t.m / 2) + r) * 8;
                    const int16_t* p = partial.data() + t.output_offset / 2 + index * 2;
                    acc_out[size_t(t.m0 / 2 + r) * N + t.n0 + n] =
                        accumulator[t.output_offset / 4 + index + n % 8] + 16 * int32_t(p[n % 8]) + p[8 + n % 8];
                }
    } else if (!rc && acc_out && !swiglu) {
        for (const auto& t : tiles)
            for (int r = 0; r < t.m / 2; ++r)
                for (int n = 0; n < t.logical_n; ++n) {
                    const size_t index = (size_t(n / 8) * (t.m / 2) + r) * 8;
                    const int16_t* p = partial.data() + t.output_offset / 2 + index * 2;
                    acc_out[size_t(t.m0 / 2 + r) * N + t.n0 + n] =
                        L.correction[t.n0 + n] + 16 * int32_t(p[n % 8]) + p[8 + n % 8];
                }
    }
    return rc;
}
} // namespace

extern "C" {

// Reference scales + codes. Codes are rebuilt from the packed high/low rows that
// w4a8_pack wrote (q = 16*high + low + 8), so this checks the reference's packing too.
int ref_quantize(const void* A, int half, int M, int K, int threads, float* scales, float* inverse, int8_t* q) {
    int rc = w4a8_scales(A, half != 0, M, K, threads, scales, inverse);
    if (rc) return rc;
    W4A8Input input{A, half != 0, M, K, scales, inverse, threads, I4InputLayout::Native};
    const int pk_all = align_to(K, 32);
    for (int k0 = 0; k0 < K; k0 += 2048) {
        const int k = std::min(2048, K - k0), pk = align_to(k, 32);
        for (int m0 = 0; m0 < M; m0 += 64) {
            const int rows = std::min(64, M - m0) * 2;
            std::vector<uint8_t> dst(size_t(rows) * pk / 2, 0);
            rk_npu_i4_input_tile tile{m0 * 2, rows, k0, k, pk, dst.data(), dst.size()};
            rc = w4a8_pack(&input, &tile);
            if (rc) return rc;
            for (int r = 0; r < rows / 2; ++r)
                for (int j = 0; j < k; ++j) {
                    const int h = nibble(dst[(size_t(j / 32) * rows + 2 * r) * 16 + (j % 32) / 2], j);
                    const int l = nibble(dst[(size_t(j / 32) * rows + 2 * r + 1) * 16 + (j % 32) / 2], j);
                    q[size_t(m0 + r) * K + k0 + j] = int8_t(16 * h + l + 8);
                }
        }
    }
    (void)pk_all;
    return RK_NPU_OK;
}

// One linear through the reference stage chain. stage_us[4]: scan, pack, stand-in, reduce.
int ref_linear(const void* A, int half, int M, int K, int N, const int8_t* B, const float* w_scale,
               int k_tile, int m_tile, int n_tile, unsigned mask, int threads, void* out,
               int32_t* acc_out, float* scales_out, int64_t* saturated, double* stage_us, double* prepare_us) {
    try {
        Layer L;
        auto t0 = Clock::now();
        int rc = prepare_layer(L, K, N, k_tile, B, w_scale);
        if (prepare_us) *prepare_us = since(t0);
        if (rc) return rc;
        std::vector<float> s(M), inv(M);
        if (saturated) *saturated = 0;
        if (stage_us) std::fill(stage_us, stage_us + 4, 0.0);
        rc = run_projection(L, {m_tile, n_tile, mask, threads}, A, half != 0, M, out, false, nullptr,
                            s.data(), inv.data(), false, acc_out, saturated, stage_us);
        if (!rc && scales_out) std::copy(s.begin(), s.end(), scales_out);
        return rc;
    } catch (...) { return RK_NPU_ERR_PARAM; }
}

// Handle-based variant so that a benchmark can exclude weight preparation,
// as the reference's own benchmark does (examples/bench_w4a8.cpp:206-228).
void* ref_layer_create(int K, int N, int k_tile, const int8_t* B, const float* w_scale) {
    try {
        auto* L = new Layer;
        if (prepare_layer(*L, K, N, k_tile, B, w_scale)) { delete L; return nullptr; }
        return L;
    } catch (...) { return nullptr; }
}
void ref_layer_free(void* layer) { delete static_cast<Layer*>(layer); }
int ref_layer_run(void* layer, const void* A, int half, int M, int m_tile, int n_tile, unsigned mask,
                  int threads, void* out, double* stage_us) {
    try {
        auto& L = *static_cast<Layer*>(layer);
        std::vector<float> s(M), inv(M);
        if (stage_us) std::fill(stage_us, stage_us + 4, 0.0);
        return run_projection(L, {m_tile, n_tile, mask, threads}, A, half != 0, M, out, false, nullptr,
                              s.data(), inv.data(), false, nullptr, nullptr, stage_us);
    } catch (...) { return RK_NPU_ERR_PARAM; }
}

// Gate/up -> fused SwiGLU (+ row maxima) -> finish scales -> down, as rk_npu_w4a8_run_ffn_f32
// (src/rk_npu_w4a8.cpp:354-380). swiglu_only stops after middle (rk_npu_w4a8_run_swiglu_f32).
int ref_ffn(const float* A, int M, int K, int F, int N, const int8_t* B_gate_up, const float* scale_gate_up,
            const int8_t* B_down, const float* scale_down, int k_tile_gate_up, int k_tile_down,
            int m_tile, int n_tile, unsigned mask, int threads, int swiglu_only, float* middle, float* C,
            float* scales_down_in, int64_t* saturated, double* stage_us) {
    try {
        Layer G, D;
        int rc = prepare_layer(G, K, 2 * F, k_tile_gate_up, B_gate_up, scale_gate_up);
        if (rc) return rc;
        std::vector<float> s(M), inv(M);
        std::vector<uint32_t> maxima(size_t(M + 16) * threads, 0u);
        if (saturated) *saturated = 0;
        if (stage_us) std::fill(stage_us, stage_us + 4, 0.0);
        rc = run_projection(G, {m_tile, n_tile, mask, threads}, A, false, M, middle, true,
                            swiglu_only ? nullptr : maxima.data(), s.data(), inv.data(), false, nullptr,
                            saturated, stage_us);
        if (rc || swiglu_only) return rc;
        rc = w4a8_finish_scales(M, threads, maxima.data(), M + 16, s.data(), inv.data());
        if (rc) return rc;
        if (scales_down_in) std::copy(s.begin(), s.end(), scales_down_in);
        rc = prepare_layer(D, F, N, k_tile_down, B_down, scale_down);
        if (rc) return rc;
        return run_projection(D, {m_tile, n_tile, mask, threads}, middle, false, M, C, false, nullptr,
                              s.data(), inv.data(), true, nullptr, saturated, stage_us);
    } catch (...) { return RK_NPU_ERR_PARAM; }
}

int ref_bound(int K, int N, const int8_t* B, int requested, int fallback, int* k_tile, int64_t* positive,
              int64_t* negative, uint64_t* safe_tiles) {
    I4WeightBound b;
    const int rc = bound_i4_weights(K, N, B, requested, b, fallback);
    if (!rc) { *k_tile = b.k_tile; *positive = b.positive; *negative = b.negative_magnitude; *safe_tiles = b.safe_tiles; }
    return rc;
}

void ref_dequant(int M, int N, const int32_t* acc, const float* a_scale, const float* w_scale, int half,
                 void* out, int threads) {
    w4a8_dequant(M, N, acc, a_scale, w_scale, half != 0, out, threads);
}
int ref_finish_scales(int M, int threads, const uint32_t* maxima, int stride, float* scales, float* inverse) {
    return w4a8_finish_scales(M, threads, maxima, stride, scales, inverse);
}
float ref_half_to_float(uint16_t h) { return rknpu2_matmul_open::bits::half_to_float(h); }
uint16_t ref_float_to_half(float f) { return rknpu2_matmul_open::bits::float_to_half(f); }
void ref_half_to_float_n(const uint16_t* src, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = rknpu2_matmul_open::bits::half_to_float(src[i]);
}
void ref_float_to_half_n(const float* src, uint16_t* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = rknpu2_matmul_open::bits::float_to_half(src[i]);
}

uint64_t ref_fingerprint(int K, int N, const int8_t* B, const float* w_scale) {
    rknpu2_matmul_open::tune::Hash hash;
    hash.mix(K); hash.mix(N);
    hash.bytes(B, size_t(K) * N); hash.bytes(w_scale, size_t(N) * sizeof(float));
    return hash.value;
}
int ref_host_threads(void) { return omp_get_max_threads(); }
// One typed W8A8 linear through the reference's own CPU stages (src/rk_npu_cpu_kernels.cpp): per-token scales,
// quantise + row-major packing, and the fused native-int32 dequantisation.  Only the device step between them --
// int8 x int8 -> int32, exact modulo 2^32, written in the device's native C layout src[((n/4)*M + m)*4 + n%4]
// (src/rk_npu_cpu_kernels.h:18-25,170-172) -- is restated here.
int ref_w8_linear(const void* A, int half, int M, int K, int N, const int8_t* B, const float* w_scale,
                  const float* a_scale_static, void* out, int32_t* acc_out, float* scales_out, int8_t* codes_out) {
    namespace cpu = rknpu2_matmul_open::cpu;
    if (!A || !B || !w_scale || !out || M < 1 || K < 1 || N < 1) return RK_NPU_ERR_PARAM;
    std::vector<float> scale(M);
    if (a_scale_static) std::copy(a_scale_static, a_scale_static + M, scale.begin());
    else if (half) cpu::i8_compute_dynamic_per_token_scale_f16(M, K, static_cast<const uint16_t*>(A), K, scale.data());
    else cpu::i8_compute_dynamic_per_token_scale_f32(M, K, static_cast<const float*>(A), K, scale.data());
    std::vector<int8_t> q(size_t(M) * K);
    if (half) cpu::i8_pack_a_f16_quant_normal_strided(M, K, K, static_cast<const uint16_t*>(A), K, scale.data(), q.data());
    else cpu::i8_pack_a_f32_quant_normal_strided(M, K, K, static_cast<const float*>(A), K, scale.data(), q.data());
    const int nb_count = (N + 3) / 4;
    std::vector<int32_t> native(size_t(nb_count) * M * 4, 0);
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            uint32_t sum = 0;
            for (int k = 0; k < K; ++k) sum += uint32_t(int32_t(q[size_t(m) * K + k]) * int32_t(B[size_t(k) * N + n]));
            native[(size_t(n / 4) * M + m) * 4 + n % 4] = int32_t(sum);
        }
    if (half) cpu::i8_unpack_c_native_i32_dequant_f16(M, N, native.data(), scale.data(), w_scale, nullptr, cpu::ActivationOp::None,
                                                      static_cast<uint16_t*>(out));
    else cpu::i8_unpack_c_native_i32_dequant_f32(M, N, native.data(), scale.data(), w_scale, nullptr, cpu::ActivationOp::None,
                                                 static_cast<float*>(out));
    if (acc_out)
        for (int m = 0; m < M; ++m)
            for (int n = 0; n < N; ++n) acc_out[size_t(m) * N + n] = native[(size_t(n / 4) * M + m) * 4 + n % 4];
    if (scales_out) std::copy(scale.begin(), scale.end(), scales_out);
    if (codes_out) std::copy(q.begin(), q.end(), codes_out);
    return RK_NPU_OK;
}
// src/rk_npu_quant_matmul.cpp:1696-1700, the public K-partition query of the reference itself
int ref_k_partition_query(int M, int K, int k_tile) { return rk_npu_matmul_k_partition_query(M, K, k_tile); }

} // extern "C"

// ---- routed experts: the reference's fused middle stage (src/rk_npu_moe_cpu.cpp:47-115) on one row of int32
// sums [gate(I), up(I)], plain int8 output.  Its x86 build evaluates the sigmoid with std::exp.
extern "C" float ref_moe_middle_row(const int32_t* acc, int I, float input_scale, const float* w_scale, int8_t* q)
{
    // W8 partial layout for one row: data[(n / 4) * rows * 4 + row * 4 + n % 4] == data[n] (src/rk_npu_moe_cpu.h:13-16)
    const rknpu2_matmul_open::moe::MiddleRow row{acc, nullptr, w_scale, input_scale, 1, 0, I, 1, 0, q,
                                                 rknpu2_matmul_open::moe::MiddleLayout::I8Normal};
    return rknpu2_matmul_open::moe::swiglu_quantize_row(row);
}
