// w8a8_kernels.cu -- weight layout and activation preparation of the typed W8A8 operators (int8 weights) on sm_100a.
//
// Reference behaviour reproduced (paths inside the reference project):
//   scales, dynamic : src/rk_npu_cpu_kernels.cpp:576-589, 626-645: s = max|x| / 127 when the maximum is positive, else 1
//                     (no lower clamp, NaN never raises the maximum, non-finite inputs are not rejected)
//   scales, static  : :590-596: the caller's per-token scale
//   codes           : :126-131: q = clamp(round_half_away(x * (1 / s)), -127, 127), NaN -> 127; a row whose scale is
//                     not positive quantises to zeros (:598-606)
//   int8 A as given : include/rk_npu_quant_matmul.h:335-340 (no quantisation at all)
// The contraction itself runs on the tcgen05 kernel of w4a8_gemm_tc.cu with int8 weights (GemmParams::w8).
//
// Weight layout  W8p[g][kb][c][r][16 B]: g = group of 32 output channels, kb = 128-element k-block, c = 16-element
// chunk of the k-block (8 of them), r = channel of the group; the 16 bytes are the int8 codes k = 128kb + 16c .. +15.
// A lane of an unpack warp (lane = channel) reads its eight 16-byte pieces of a k-block 512 bytes apart, so a warp's
// loads are conflict free, and the pieces are the words of that channel's tensor-memory row in order.
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"

namespace rkb200 {

__global__ void __launch_bounds__(256) w8_pack_weights_kernel(const W8PackParams p)
{
    // one thread per 32-bit word: four consecutive k of one channel; consecutive threads take consecutive channels
    const long long total = (long long)p.NG * p.KB * 8 * 4 * GROUP;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int r = (int)(idx % GROUP);
    long long rest = idx / GROUP;
    const int j = (int)(rest % 4);
    rest /= 4;
    const int c = (int)(rest % (p.KB * 8));      // 16-element chunk over all of K
    const int g = (int)(rest / (p.KB * 8));
    const int n = g * GROUP + r;
    uint32_t word = 0;
    if (n < p.N) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int k = c * 16 + 4 * j + b;
            if (k < p.K) word |= (uint32_t)(uint8_t)p.B[(size_t)k * p.N + n] << (8 * b);
        }
    }
    reinterpret_cast<uint32_t*>(p.Wp)[(((size_t)g * p.KB * 8 + c) * GROUP + r) * 4 + j] = word;
}

cudaError_t launch_w8_pack_weights(const W8PackParams& p, cudaStream_t stream)
{
    const long long total = (long long)p.NG * p.KB * 8 * 4 * GROUP;
    w8_pack_weights_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(p);
    return cudaGetLastError();
}

// round_half_away + clamp of one product; NaN gives +127 like the reference's min/max chain
__device__ __forceinline__ int w8_code(float x, float inv)
{
    const float y = __fmul_rn(x, inv);
    return (y != y) ? 127 : round_clamp(y);
}

// One CTA per token: scale (dynamic scan or the caller's), then codes in the Xq layout.  MODE 0 dynamic, 1 static.
template <bool HALF>
__global__ void __launch_bounds__(256) w8_quantize_kernel(const W8QuantParams p)
{
    using T = typename ActType<HALF>::type;
    const int m = blockIdx.x, tid = threadIdx.x;
    const T* row = reinterpret_cast<const T*>(p.A) + (size_t)m * p.K;
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const int chunks = p.Kp / 16, live_chunks = (p.K + 15) / 16;
    __shared__ uint32_t s_part[8];
    __shared__ float s_scale;
    if (p.static_scale == nullptr) {
        // magnitude bits order like magnitudes; a NaN pattern (above infinity) never raises the maximum
        constexpr uint32_t INF = HALF ? 0x7c00u : 0x7f800000u;
        uint32_t best = 0;
        for (int kc = tid; kc < live_chunks; kc += 256) {
            Raw16<HALF> r;
            load_raw<HALF>(row, kc * 16, p.K, vec, r);
            if constexpr (HALF) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t lo = r.w[i] & 0x7fffu, hi = (r.w[i] >> 16) & 0x7fffu;
                    if (lo <= INF) best = max(best, lo);
                    if (hi <= INF) best = max(best, hi);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t a = r.w[i] & 0x7fffffffu;
                    if (a <= INF) best = max(best, a);
                }
            }
        }
        best = __reduce_max_sync(0xffffffffu, best);
        if ((tid & 31) == 0) s_part[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            uint32_t mx = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) mx = max(mx, s_part[i]);
            float maximum;
            if constexpr (HALF) maximum = __half2float(__ushort_as_half((uint16_t)mx));
            else maximum = __uint_as_float(mx);
            const float s = maximum > 0.f ? __fdiv_rn(maximum, 127.0f) : 1.0f;
            s_scale = s;
            p.scales[m] = s;
        }
    } else if (tid == 0) {
        const float s = p.static_scale[m];
        s_scale = s;
        p.scales[m] = s;
    }
    __syncthreads();
    const float s = s_scale;
    const bool live = s > 0.f;                       // a scale that is not positive (an underflowed maximum) gives zeros
    const float inv = live ? __fdiv_rn(1.0f, s) : 0.f;
    const int mt = m / p.T, t = m - mt * p.T;
    uint4* dst = reinterpret_cast<uint4*>(p.Xq) + ((size_t)mt * chunks) * p.T + t;
    for (int kc = tid; kc < chunks; kc += 256) {
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        if (live && kc < live_chunks) {
            Raw16<HALF> r;
            float v[16];
            load_raw<HALF>(row, kc * 16, p.K, vec, r);
            raw_to_float<HALF>(r, v);
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int k = kc * 16 + 4 * j + i;
                    const int q = k < p.K ? w8_code(v[4 * j + i], inv) : 0;
                    w[j] |= (uint32_t)(q & 0xff) << (8 * i);
                }
        }
        dst[(size_t)kc * p.T] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// int8 activations as given -> the Xq layout; every token's scale is 1
__global__ void __launch_bounds__(256) w8_codes_kernel(const W8QuantParams p)
{
    const int m = blockIdx.x, tid = threadIdx.x;
    const int8_t* row = reinterpret_cast<const int8_t*>(p.A) + (size_t)m * p.K;
    const int chunks = p.Kp / 16;
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const int mt = m / p.T, t = m - mt * p.T;
    uint4* dst = reinterpret_cast<uint4*>(p.Xq) + ((size_t)mt * chunks) * p.T + t;
    if (tid == 0) p.scales[m] = 1.0f;
    for (int kc = tid; kc < chunks; kc += 256) {
        uint4 q = make_uint4(0u, 0u, 0u, 0u);
        const int k0 = kc * 16;
        if (vec && k0 + 16 <= p.K) q = *reinterpret_cast<const uint4*>(row + k0);
        else {
            uint32_t w[4] = {0u, 0u, 0u, 0u};
            for (int i = 0; i < 16; ++i)
                if (k0 + i < p.K) w[i >> 2] |= (uint32_t)(uint8_t)row[k0 + i] << (8 * (i & 3));
            q = make_uint4(w[0], w[1], w[2], w[3]);
        }
        dst[(size_t)kc * p.T] = q;
    }
}

cudaError_t launch_w8_quantize(const W8QuantParams& p, cudaStream_t stream)
{
    if (p.M < 1 || p.T < 1) return cudaErrorInvalidValue;
    if (p.kind == 2) w8_codes_kernel<<<(unsigned)p.M, 256, 0, stream>>>(p);
    else if (p.kind == 1) w8_quantize_kernel<true><<<(unsigned)p.M, 256, 0, stream>>>(p);
    else w8_quantize_kernel<false><<<(unsigned)p.M, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

} // namespace rkb200
