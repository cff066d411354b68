// w4a8_kernels.cu -- weight repacking, per-token activation quantisation and the
// mma.sync W4A8 GEMM (decode / small-batch path and general fallback) for sm_100a.
//
// Reference behaviour reproduced (paths inside the reference project):
//   quantise_kernel : src/rk_npu_w4a8_quant.cpp:52-85 (scales), :119-121 (codes),
//                     :145-161 (scales from collected row maxima)
//   gemm epilogues  : src/rk_npu_w4a8_output.cpp:70-76 (dequantise),
//                     src/rk_npu_w4a8_swiglu.cpp:12-91 + src/rk_npu_swiglu_fp32_neon.h:13-51
//   pack_weights    : src/rk_npu_w4a8.cpp:236-242 (code range check); layout is new.
#include "w4a8_device.h"
#include "w4a8_host.h"
#include "w4a8_ptx.cuh"
#include "w4a8_math.cuh"
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <float.h>

namespace cg = cooperative_groups;

namespace rkb200 {

// =============================================================== weight repacking
// One thread builds one 32-bit word of the packed layout: eight codes of one output
// channel.  Consecutive threads take consecutive channels so the reads of B[k, :] are
// coalesced; the 4-byte writes of a warp land 16 bytes apart and are merged in L2.
__global__ void __launch_bounds__(256) pack_weights_kernel(const PackParams p)
{
    const long long total = (long long)p.NG * p.KC * 4 * GROUP;
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int r = (int)(idx % GROUP);
    long long rest = idx / GROUP;
    const int j = (int)(rest % 4);
    rest /= 4;
    const int c = (int)(rest % p.KC);
    const int g = (int)(rest / p.KC);
    const int n = g * GROUP + r;
    uint32_t word = 0;
    int bad = 0;
    if (n < p.N) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int k_lo = c * 32 + 4 * j + b, k_hi = k_lo + 16;
            int lo = 0, hi = 0;
            if (k_lo < p.K) lo = p.B[(size_t)k_lo * p.N + n];
            if (k_hi < p.K) hi = p.B[(size_t)k_hi * p.N + n];
            bad |= (lo < -8) | (lo > 7) | (hi < -8) | (hi > 7);
            word |= (uint32_t)((lo & 15) | ((hi & 15) << 4)) << (8 * b);
        }
    }
    if (bad) atomicOr(p.error, 1);
    reinterpret_cast<uint32_t*>(p.Wp)[(((size_t)g * p.KC + c) * GROUP + r) * 4 + j] = word;
}

cudaError_t launch_pack_weights(const PackParams& p, cudaStream_t stream)
{
    const long long total = (long long)p.NG * p.KC * 4 * GROUP;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    pack_weights_kernel<<<blocks, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

// =============================================================== activation quantisation
// One CTA per token.  Pass 1: max |x| over the full row on the raw bit patterns (for
// binary16 and fp32 alike the magnitude bits order like the magnitudes, and anything
// at or above the infinity pattern is NaN/Inf).  Pass 2: q = clamp(round_half_away(
// x * inverse), -127, 127), written as 16-byte units of the Xq layout.
template <bool HALF, int BS>
__global__ void __launch_bounds__(BS, 2048 / BS) quantize_kernel(const QuantParams p)
{
    using T = typename ActType<HALF>::type;
    pdl_launch_dependents();   // the GEMM behind this kernel may start prefetching weights
    pdl_wait();                // A may be the output of the kernel in front of this one
    const int m = blockIdx.x, tid = threadIdx.x;
    const T* row = reinterpret_cast<const T*>(p.A) + (size_t)m * p.K;
    const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
    const int chunks = p.Kp / 16, live_chunks = (p.K + 15) / 16;
    __shared__ uint32_t s_part[BS / 32];
    __shared__ float s_inverse;
    __shared__ int s_bad;

    uint32_t maxbits = 0;
    int bad = 0;
    if (p.rowmax == nullptr) {
        float v[16];
        for (int kc = tid; kc < live_chunks; kc += BS) load16<HALF>(row, kc * 16, p.K, vec, v, maxbits);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) maxbits = max(maxbits, __shfl_xor_sync(0xffffffffu, maxbits, o));
        if ((tid & 31) == 0) s_part[tid >> 5] = maxbits;
        __syncthreads();
        if (tid == 0) {
            uint32_t mx = 0;
#pragma unroll
            for (int i = 0; i < BS / 32; ++i) mx = max(mx, s_part[i]);
            float maximum;
            if constexpr (HALF) {
                bad = mx >= 0x7c00u ? 1 : 0;
                maximum = __half2float(__ushort_as_half((uint16_t)mx));
            } else {
                bad = mx >= 0x7f800000u ? 1 : 0;
                maximum = __uint_as_float(mx);
            }
            const float s = (maximum == 0.f || bad) ? 1.0f : fmaxf(__fdiv_rn(maximum, 127.0f), FLT_MIN);
            const float inv = __fdiv_rn(1.0f, s);
            p.scales[m] = s;
            p.inverse[m] = inv;
            s_inverse = inv;
            s_bad = bad;
        }
    } else if (tid == 0) {
        const uint32_t bits = p.rowmax[m];
        p.rowmax[m] = 0u;   // consumed: the next SwiGLU epilogue maxes into a clean word
        bad = bits >= 0x7f800000u ? 2 : 0;
        const float maximum = __uint_as_float(bits);
        const float s = (maximum == 0.f || bad) ? 1.0f : fmaxf(__fdiv_rn(maximum, 127.0f), FLT_MIN);
        const float inv = __fdiv_rn(1.0f, s);
        p.scales[m] = s;
        p.inverse[m] = inv;
        s_inverse = inv;
        s_bad = bad;
    }
    __syncthreads();
    const float inv = s_inverse;
    const int mt = m / p.T, t = m - mt * p.T;
    uint4* dst = reinterpret_cast<uint4*>(p.Xq) + ((size_t)mt * chunks) * p.T + t;
    // (the row is read a second time here, from L2: keeping it in registers between the passes needs more than the 32
    // registers per thread that let sixteen 128-thread CTAs share an SM -- the compiler spilled it)
    for (int kc = tid; kc < chunks; kc += BS) {
        uint4 q = make_uint4(0u, 0u, 0u, 0u);
        if (kc < live_chunks) {
            float v[16];
            uint32_t unused = 0;
            load16<HALF>(row, kc * 16, p.K, vec, v, unused);
            q = quantize16(v, inv, kc * 16, p.K);
        }
        dst[(size_t)kc * p.T] = q;
    }
    // Cross-CTA bookkeeping last, so that the other 255 threads of the CTA never wait for its
    // round trips to L2.
    if (tid == 0) {
        if (p.rowmax_zero) p.rowmax_zero[m] = 0u;
        // "Any row bad" across CTAs without a reset pass: the last CTA to arrive
        // publishes the accumulated flag and clears the scratch word; the counter
        // wraps to zero by itself (atomicInc with limit M-1).
        if (gridDim.x == 1) {
            // a single row: its verdict is the verdict, no round trips through L2 before the kernel can end
            p.status->bad_input = bad;
            if (p.host_flag) *p.host_flag = bad;
        } else {
            if (bad) atomicOr(&p.status->bad_accum, bad);
            __threadfence();
            const unsigned prev = atomicInc(&p.status->done, (unsigned)p.M - 1u);
            if (prev == (unsigned)p.M - 1u) {
                __threadfence();
                const int any = atomicExch(&p.status->bad_accum, 0);
                p.status->bad_input = any;
                if (p.host_flag) *p.host_flag = any;
            }
        }
    }
}

cudaError_t launch_quantize(const QuantParams& p, cudaStream_t stream, bool pdl)
{
    cudaLaunchConfig_t cfg = {};
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    // One CTA per token.  With many tokens the kernel is bound by how many rows are in flight, so
    // rows of up to 4096 elements get 128-thread CTAs (16 resident per SM instead of 8).
    const bool narrow = p.M >= 512 && p.K <= 4096;
    cfg.gridDim = dim3((unsigned)p.M);
    cfg.blockDim = dim3(narrow ? 128 : 256);
    cfg.dynamicSmemBytes = 0;
    if (narrow) return p.half ? cudaLaunchKernelEx(&cfg, quantize_kernel<true, 128>, p) : cudaLaunchKernelEx(&cfg, quantize_kernel<false, 128>, p);
    return p.half ? cudaLaunchKernelEx(&cfg, quantize_kernel<true, 256>, p) : cudaLaunchKernelEx(&cfg, quantize_kernel<false, 256>, p);
}

// =============================================================== mma.sync GEMM
// Output-stationary, swap-AB: the 128 output channels of a CTA are the M side of
// mma.m16n8k32 (weights = A fragments built from the packed nibbles with three ALU
// instructions per eight codes), the tokens are the N side (8 per instruction).
// One producer thread streams weight and activation k-blocks with bulk async copies
// into a ring of stages; four consumer warps (one weight group each) do the math.
// Split-K runs as a thread-block cluster along y: partial sums are exchanged through
// distributed shared memory, each rank finishing a slice of the channels.
constexpr int MMA_STAGES = 8;
constexpr int RED_STRIDE = 132;   // int32 words per token row of the reduction buffer

__host__ __device__ constexpr int mma_stage_bytes(int tc) { return 4 * 2048 + 128 * tc; }
__host__ __device__ constexpr size_t mma_smem_bytes(int tc)
{
    return (size_t)MMA_STAGES * mma_stage_bytes(tc) + (size_t)tc * RED_STRIDE * 4 + 2 * MMA_STAGES * 8 + 16;
}
size_t gemm_mma_smem_bytes(int tokens_per_cta) { return mma_smem_bytes(tokens_per_cta); }

template <int NT, bool BIGK>
__global__ void __launch_bounds__(160, 1) gemm_mma_kernel(const GemmParams p)
{
    constexpr int TC = 8 * NT;
    constexpr int XB = 128 * TC;
    constexpr int STAGE = mma_stage_bytes(TC);
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* const stages = smem;
    int32_t* const red = reinterpret_cast<int32_t*>(smem + MMA_STAGES * STAGE);
    uint64_t* const full = reinterpret_cast<uint64_t*>(smem + MMA_STAGES * STAGE + TC * RED_STRIDE * 4);
    uint64_t* const empty = full + MMA_STAGES;

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, rank = blockIdx.y, S = p.split;
    const int tok0 = blockIdx.z * TC;
    const bool swiglu = p.epi == EPI_SWIGLU;
    const int KC = p.KB * 4;
    const int kb0 = (int)(((long long)p.KB * rank) / S), kb1 = (int)(((long long)p.KB * (rank + 1)) / S);
    const int nkb = kb1 - kb0;
    const unsigned long long deadline = global_ns() + p.timeout_ns;

    if (tid == 0) {
        for (int s = 0; s < MMA_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 4); }
        mbar_fence_init();
    }
    __syncthreads();

    int acc[2][NT][4];
    int hi[BIGK ? 2 : 1][BIGK ? NT : 1][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[a][j][e] = 0;
    if constexpr (BIGK) {
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) hi[a][j][e] = 0;
    }

    if (warp == 4) {
        if (lane == 0) {
            // ---------------- producer
            int group[4];
#pragma unroll
            for (int w = 0; w < 4; ++w)
                group[w] = swiglu ? (w < 2 ? tile * 2 + w : p.F / GROUP + tile * 2 + (w - 2)) : tile * 4 + w;
            const int mt = tok0 / p.T, r0 = tok0 - mt * p.T;
            const size_t kc16_total = (size_t)p.KB * 8;
            auto copy_w = [&](int it, int s) {
#pragma unroll
                for (int w = 0; w < 4; ++w)
                    bulk_g2s(stages + (size_t)s * STAGE + w * 2048,
                             p.Wp + ((size_t)group[w] * KC + (size_t)(kb0 + it) * 4) * 512, 2048, &full[s]);
            };
            auto copy_x = [&](int it, int s) {
                uint8_t* dst = stages + (size_t)s * STAGE + 8192;
                const size_t kc16 = (size_t)(kb0 + it) * 8;
                if (p.T == TC) {
                    bulk_g2s(dst, p.Xq + ((size_t)mt * kc16_total + kc16) * p.T * 16, XB, &full[s]);
                } else {
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        bulk_g2s(dst + c * TC * 16, p.Xq + (((size_t)mt * kc16_total + kc16 + c) * p.T + r0) * 16,
                                 TC * 16, &full[s]);
                }
            };
            const int pre = nkb < MMA_STAGES ? nkb : MMA_STAGES;
            // Weights never change, so their first stages are requested before waiting
            // for the kernel in front (which produces the activation codes).
            for (int it = 0; it < pre; ++it) { mbar_expect_tx(&full[it], 8192); copy_w(it, it); }
            pdl_wait();
            const bool skip = *reinterpret_cast<volatile const int*>(&p.status->bad_input) != 0;
            for (int it = 0; it < pre; ++it) {
                if (skip) { mbar_arrive(&full[it]); }
                else { mbar_arrive_expect_tx(&full[it], XB); copy_x(it, it); }
            }
            if (!skip) {
                for (int it = pre; it < nkb; ++it) {
                    const int s = it % MMA_STAGES;
                    if (!mbar_wait(&empty[s], ((it / MMA_STAGES) - 1) & 1, deadline)) {
                        atomicExch(&p.status->device_error, 1);
                        break;
                    }
                    mbar_arrive_expect_tx(&full[s], STAGE);
                    copy_w(it, s);
                    copy_x(it, s);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- consumers: warp w owns weight group w (32 channels = two m16 tiles)
        pdl_wait();
        const bool skip = *reinterpret_cast<volatile const int*>(&p.status->bad_input) != 0;
        const int iters = skip ? (nkb < MMA_STAGES ? nkb : MMA_STAGES) : nkb;
        const int g8 = lane >> 2, t4 = lane & 3;
        for (int it = 0; it < iters; ++it) {
            const int s = it % MMA_STAGES;
            if (!mbar_wait(&full[s], (it / MMA_STAGES) & 1, deadline)) {
                if (lane == 0) atomicExch(&p.status->device_error, 1);
                break;
            }
            if (!skip) {
                const uint32_t wbase = smem_u32(stages + (size_t)s * STAGE + warp * 2048) + g8 * 16 + t4 * 4;
                const uint32_t xbase = smem_u32(stages + (size_t)s * STAGE + 8192) + g8 * 16 + t4 * 4;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t a[2][4];
#pragma unroll
                    for (int mtile = 0; mtile < 2; ++mtile) {
                        const uint32_t w0 = lds32(wbase + (c * 32 + mtile * 16) * 16);
                        const uint32_t w1 = lds32(wbase + (c * 32 + mtile * 16 + 8) * 16);
                        a[mtile][0] = (w0 << 4) & 0xF0F0F0F0u;
                        a[mtile][1] = (w1 << 4) & 0xF0F0F0F0u;
                        a[mtile][2] = w0 & 0xF0F0F0F0u;
                        a[mtile][3] = w1 & 0xF0F0F0F0u;
                    }
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        const uint32_t b0 = lds32(xbase + ((2 * c) * TC + 8 * j) * 16);
                        const uint32_t b1 = lds32(xbase + ((2 * c + 1) * TC + 8 * j) * 16);
                        mma_s8(acc[0][j], a[0][0], a[0][1], a[0][2], a[0][3], b0, b1);
                        mma_s8(acc[1][j], a[1][0], a[1][1], a[1][2], a[1][3], b0, b1);
                    }
                }
                if constexpr (BIGK) {
                    // 16*|sum| stays below 2^31 for 512 k-blocks; fold the exact quotient away.
                    if ((it & 511) == 511) {
#pragma unroll
                        for (int a = 0; a < 2; ++a)
#pragma unroll
                            for (int j = 0; j < NT; ++j)
#pragma unroll
                                for (int e = 0; e < 4; ++e) { hi[a][j][e] += acc[a][j][e] >> 4; acc[a][j][e] = 0; }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        // partial sums -> reduction buffer [token][channel]
#pragma unroll
        for (int mtile = 0; mtile < 2; ++mtile)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int v = acc[mtile][j][e] >> 4;
                    if constexpr (BIGK) v += hi[mtile][j][e];
                    const int ch = warp * 32 + mtile * 16 + g8 + (e >> 1) * 8;
                    const int tok = 8 * j + 2 * t4 + (e & 1);
                    red[tok * RED_STRIDE + ch] = v;
                }
    }
    __syncthreads();
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync();

    const bool skip_out = *reinterpret_cast<volatile const int*>(&p.status->bad_input) != 0;
    if (tid < 128 && !skip_out) {
        const int CH = (swiglu ? 64 : 128) / S;       // channels (gate channels) this rank finishes
        const int IPT = CH / 4;                       // 4-channel items per token
        const int items = TC * IPT;
        for (int base = 0; base < items; base += 128) {
            const int i = base + tid;
            const bool active = i < items;
            const int tok = active ? i / IPT : 0, c4 = active ? i - tok * IPT : 0;
            const int ch = rank * CH + c4 * 4;
            const int m = tok0 + tok;
            int4 v = make_int4(0, 0, 0, 0), u = make_int4(0, 0, 0, 0);
            if (active) {
                for (int q = 0; q < S; ++q) {
                    const int32_t* src = S > 1 ? cluster.map_shared_rank(red, q) : red;
                    const int4 a = *reinterpret_cast<const int4*>(src + tok * RED_STRIDE + ch);
                    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                    if (swiglu) {
                        const int4 b = *reinterpret_cast<const int4*>(src + tok * RED_STRIDE + 64 + ch);
                        u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
                    }
                }
            }
            const bool row_ok = active && m < p.M;
            if (!swiglu) {
                const int n = tile * TILE_N + ch;
                if (row_ok && n < p.N) {
                    const int va[4] = {v.x, v.y, v.z, v.w};
                    if (p.epi == EPI_I32) {
                        int* out = reinterpret_cast<int*>(p.out) + (size_t)m * p.N + n;
                        if (n + 3 < p.N && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) *reinterpret_cast<int4*>(out) = v;
                        else for (int e = 0; e < 4; ++e) if (n + e < p.N) out[e] = va[e];
                    } else {
                        const float sx = p.sx[m];
                        float y[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) y[e] = dequant(va[e], sx, p.sw[n + e]);
                        if (p.epi == EPI_F32) {
                            float* out = reinterpret_cast<float*>(p.out) + (size_t)m * p.N + n;
                            if (n + 3 < p.N && (reinterpret_cast<uintptr_t>(out) & 15u) == 0)
                                *reinterpret_cast<float4*>(out) = make_float4(y[0], y[1], y[2], y[3]);
                            else for (int e = 0; e < 4; ++e) if (n + e < p.N) out[e] = y[e];
                        } else {
                            __half* out = reinterpret_cast<__half*>(p.out) + (size_t)m * p.N + n;
                            if (n + 3 < p.N && (reinterpret_cast<uintptr_t>(out) & 7u) == 0) {
                                const __half2 h0 = __halves2half2(__float2half_rn(y[0]), __float2half_rn(y[1]));
                                const __half2 h1 = __halves2half2(__float2half_rn(y[2]), __float2half_rn(y[3]));
                                uint2 pk;
                                pk.x = *reinterpret_cast<const uint32_t*>(&h0);
                                pk.y = *reinterpret_cast<const uint32_t*>(&h1);
                                *reinterpret_cast<uint2*>(out) = pk;
                            } else for (int e = 0; e < 4; ++e) if (n + e < p.N) out[e] = __float2half_rn(y[e]);
                        }
                    }
                }
            } else {
                const int f = tile * 64 + ch;
                uint32_t mx = 0;
                if (row_ok && f < p.F) {
                    const float sx = p.sx[m];
                    const int ga[4] = {v.x, v.y, v.z, v.w}, ua[4] = {u.x, u.y, u.z, u.w};
                    float y[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float g = dequant(ga[e], sx, p.sw[f + e]);
                        const float up = dequant(ua[e], sx, p.sw[p.F + f + e]);
                        y[e] = __fmul_rn(silu_poly(g), up);
                        mx = max(mx, __float_as_uint(y[e]) & 0x7fffffffu);
                    }
                    float* out = reinterpret_cast<float*>(p.out) + (size_t)m * p.F + f;
                    if ((reinterpret_cast<uintptr_t>(out) & 15u) == 0) *reinterpret_cast<float4*>(out) = make_float4(y[0], y[1], y[2], y[3]);
                    else for (int e = 0; e < 4; ++e) out[e] = y[e];
                }
                if (p.rowmax) {
                    // lanes of an aligned group of IPT share the token: one atomic per group
                    for (int o = 1; o < IPT && o < 32; o <<= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    if (row_ok && (lane & (IPT - 1) & 31) == 0 && mx) atomicMax(&p.rowmax[m], mx);
                }
            }
        }
    }
    if (S > 1) cluster.sync();   // nobody leaves while a peer may still read its partials
}

template <int NT, bool BIGK>
static cudaError_t launch_mma_inst(const GemmParams& p, cudaStream_t stream, bool pdl)
{
    constexpr int TC = 8 * NT;
    const size_t smem = mma_smem_bytes(TC);
    static PerDeviceOnce configured;
    int configured_device = -1;
    auto kernel = gemm_mma_kernel<NT, BIGK>;
    if (configured.needed(configured_device)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured.mark(configured_device);
    }
    const int tiles = p.epi == EPI_SWIGLU ? (p.F + 63) / 64 : (p.N + TILE_N - 1) / TILE_N;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles, (unsigned)p.split, (unsigned)((p.M + TC - 1) / TC));
    cfg.blockDim = dim3(160);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = (unsigned)p.split;
    attr[n].val.clusterDim.z = 1;
    ++n;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

cudaError_t launch_gemm_mma(const GemmParams& p, int tokens_per_cta, cudaStream_t stream, bool pdl)
{
    if (p.split != 1 && p.split != 2 && p.split != 4 && p.split != 8) return cudaErrorInvalidValue;
    if (p.T % tokens_per_cta) return cudaErrorInvalidValue;
    const bool big = (long long)p.KB * KBLOCK > 131072;
    switch (tokens_per_cta) {
    case 8: return big ? launch_mma_inst<1, true>(p, stream, pdl) : launch_mma_inst<1, false>(p, stream, pdl);
    case 16: return big ? launch_mma_inst<2, true>(p, stream, pdl) : launch_mma_inst<2, false>(p, stream, pdl);
    case 32: return big ? launch_mma_inst<4, true>(p, stream, pdl) : launch_mma_inst<4, false>(p, stream, pdl);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace rkb200

// =============================================================== linear without any allocation
// Some callers may not allocate at the moment they need a linear: an inference engine that
// sized its one device pool at start-up and forbids cudaMalloc afterwards, a plugin running
// inside somebody else's real-time loop, code on a path where an allocation (and the implicit
// device synchronisation cudaMalloc and cudaFree bring) is not acceptable.  A workspace is
// what normally owns the scratch of a call -- the quantised activation codes, the per-token
// scales and the status word -- and creating one allocates.  The entry point below runs the
// same two kernels as a small-batch workspace (quantise, then the mma.sync split-K GEMM) with
// that scratch in a fixed array that is part of the library image, so the call itself
// allocates nothing.  Every GPU that loads the library carries the array until exit.
namespace {
constexpr int STATIC_MAX_TOKENS = 32;
constexpr size_t STATIC_CODE_BYTES = size_t(2) << 20;               // activation codes: tokens_per_cta x padded K bytes
constexpr size_t STATIC_SCRATCH_BYTES = STATIC_CODE_BYTES + 4096;   // + scales, inverse scales, status block
}
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_lock;
unsigned char* g_static_ptr[64] = {};   // device address of the array, per CUDA ordinal

// The array's name is only a host-side handle; kernels need its address on the current device.
int static_scratch(int device, unsigned char** out)
{
    if (device < 0 || device >= 64) return RK_NPU_ERR_PARAM;
    std::lock_guard<std::mutex> guard(g_static_lock);
    if (!g_static_ptr[device]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) { cudaGetLastError(); return RK_NPU_ERR_IOCTL; }
        g_static_ptr[device] = static_cast<unsigned char*>(ptr);
    }
    *out = g_static_ptr[device];
    return RK_NPU_OK;
}
} // namespace

namespace {
// Makes `device` current for the duration of a call and restores what the caller had.
struct DeviceScope {
    int previous = -1;
    bool ok = false;
    explicit DeviceScope(int device)
    {
        if (cudaGetDevice(&previous) != cudaSuccess) { cudaGetLastError(); previous = -1; }
        ok = previous == device || cudaSetDevice(device) == cudaSuccess;
        if (!ok) cudaGetLastError();
        if (previous == device) previous = -1;
    }
    ~DeviceScope() { if (previous >= 0) cudaSetDevice(previous); }
};
} // namespace

// What the last allocation-free linear on `weights`' GPU left in the array's status block.  Copies 16 bytes
// into the caller's variables; allocates nothing.  The caller has synchronised the stream of that call.
extern "C" int rk_npu_b200_w4a8_static_status(const rk_npu_w4a8_weights* weights, int* bad_input, int* device_error)
{
    using namespace rkb200;
    if (!weights || !bad_input || !device_error) return RK_NPU_ERR_PARAM;
    const rk_npu_ctx* ctx = weights->domain->ctx;
    DeviceScope scope(ctx->device);
    if (!scope.ok) return RK_NPU_ERR_SUBMIT;
    unsigned char* base = nullptr;
    const int rc = static_scratch(ctx->device, &base);
    if (rc) return rc;
    Status host{};
    if (cudaMemcpy(&host, base + STATIC_CODE_BYTES + 1024, sizeof(Status), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return RK_NPU_ERR_SUBMIT;
    }
    *bad_input = host.bad_input;
    *device_error = host.device_error;
    return host.device_error ? RK_NPU_ERR_SUBMIT : host.bad_input ? RK_NPU_ERR_PARAM : RK_NPU_OK;
}

extern "C" int rk_npu_b200_w4a8_enqueue_f16_static(const rk_npu_w4a8_weights* weights, const uint16_t* dA, uint16_t* dC,
                                                   int M, void* cuda_stream)
{
    using namespace rkb200;
    if (!weights || !dA || !dC || dA == dC || M < 1) return RK_NPU_ERR_PARAM;
    const int K = weights->info.config.K, N = weights->info.config.N;
    const int tokens = M <= 8 ? 8 : M <= 16 ? 16 : 32;
    const size_t code_bytes = size_t(tokens) * weights->KB * KBLOCK;
    // sizes beyond the fixed array are refused, never truncated
    if (M > STATIC_MAX_TOKENS || code_bytes > STATIC_CODE_BYTES) return RK_NPU_ERR_NOMEM;
    const rk_npu_ctx* ctx = weights->domain->ctx;
    if (ctx->world > 1) return RK_NPU_ERR_PARAM;   // sharded weights: the exchange behind a group linear needs a workspace
    DeviceScope scope(ctx->device);   // the caller's current device is put back on return
    if (!scope.ok) return RK_NPU_ERR_SUBMIT;
    unsigned char* base = nullptr;
    const int rc = static_scratch(ctx->device, &base);
    if (rc) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    uint8_t* codes = base;
    float* scales = reinterpret_cast<float*>(base + STATIC_CODE_BYTES);
    Status* status = reinterpret_cast<Status*>(base + STATIC_CODE_BYTES + 1024);
    // The array keeps whatever the previous call left: padding rows of the code tile and the
    // status block must start at zero.
    if (cudaMemsetAsync(codes, 0, code_bytes, stream) != cudaSuccess ||
        cudaMemsetAsync(status, 0, sizeof(Status), stream) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    QuantParams q{};
    q.A = dA;
    q.Xq = codes;
    q.scales = scales;
    q.inverse = scales + STATIC_MAX_TOKENS;
    q.status = status;
    q.M = M;
    q.K = K;
    q.Kp = weights->KB * KBLOCK;
    q.T = tokens;
    q.half = 1;
    if (launch_quantize(q, stream, false) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    GemmParams g{};
    g.Wp = weights->packed;
    g.Xq = codes;
    g.sx = scales;
    g.sw = weights->scales;
    g.out = dC;
    g.status = status;
    g.M = M;
    g.N = N;
    g.K = K;
    g.KB = weights->KB;
    g.NG = weights->NG;
    g.T = tokens;
    g.epi = EPI_F16;
    g.timeout_ns = 500ull * 1000000ull;
    const int tiles = (N + TILE_N - 1) / TILE_N;
    int split = 1;
    while (split < 8 && (long long)tiles * split * 2 <= (long long)(5 * ctx->sm_count) / 2 && weights->KB / (split * 2) >= 2) split *= 2;
    g.split = split;
    if (launch_gemm_mma(g, tokens, stream, false) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    return RK_NPU_OK;
}
