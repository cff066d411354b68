// w4a8_shard.cu -- the two kernels a column-sharded FFN puts around its exchange.
//
// With the FFN split over several GPUs each one holds a feature slice middle[:, f0:f1] of the
// SwiGLU output, but the down projection contracts over all of F and its per-token scale is
// max|middle[m, :]| / 127 over the whole row.  Row maxima are exact under any grouping (a
// maximum is a maximum), so the GPUs combine their slice maxima, quantise their own slice with
// the combined scale and exchange the int8 codes -- a quarter of the bytes of the fp32 middle --
// and every GPU ends up with exactly the codes the single-GPU quantiser produces
// (src/rk_npu_w4a8_quant.cpp:31-49 for the code rule, :145-161 for the scale from the maxima).
//
//   quantize_slice_kernel   middle slice [M, cols] fp32 + row maxima -> int8 codes [M, cols]
//   codes_in_kernel         gathered codes [parts][M][K/parts] + row maxima -> the Xq layout,
//                           per-token scales, and the bad-input verdict the GEMM reads
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"

namespace rkb200 {

namespace {
// The scale rule of the down projection's own quantiser for a row whose maximum is known.
__device__ __forceinline__ float scale_from_bits(uint32_t bits, int& bad)
{
    bad = bits >= 0x7f800000u ? 2 : 0;
    const float maximum = __uint_as_float(bits);
    return (maximum == 0.f || bad) ? 1.0f : fmaxf(__fdiv_rn(maximum, 127.0f), FLT_MIN);
}
}

__global__ void __launch_bounds__(256, 8) quantize_slice_kernel(const SliceQuantParams p)
{
    const int m = blockIdx.x, tid = threadIdx.x;
    int bad;
    const float inv = __fdiv_rn(1.0f, scale_from_bits(p.rowmax[m], bad));
    const float* row = p.X + (size_t)m * p.cols;
    int8_t* out = p.codes + (size_t)m * p.cols;
    const bool vec_in = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const bool vec_out = (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    const int chunks = (p.cols + 15) / 16;
    for (int kc = tid; kc < chunks; kc += 256) {
        float v[16];
        uint32_t unused = 0;
        load16<false>(row, kc * 16, p.cols, vec_in, v, unused);
        const uint4 q = quantize16(v, inv, kc * 16, p.cols);
        if (vec_out && kc * 16 + 16 <= p.cols) {
            *reinterpret_cast<uint4*>(out + kc * 16) = q;
        } else {
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            for (int i = 0; i < 16 && kc * 16 + i < p.cols; ++i) out[kc * 16 + i] = (int8_t)((w[i >> 2] >> (8 * (i & 3))) & 0xffu);
        }
    }
}

cudaError_t launch_quantize_slice(const SliceQuantParams& p, cudaStream_t stream)
{
    quantize_slice_kernel<<<(unsigned)p.M, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

__global__ void __launch_bounds__(256, 8) codes_in_kernel(const CodesInParams p)
{
    pdl_launch_dependents();   // the GEMM behind this kernel may start prefetching weights
    const int m = blockIdx.x, tid = threadIdx.x;
    const int chunks = p.Kp / 16, live_chunks = (p.K + 15) / 16;
    const int pc = p.K / p.parts;   // columns per part; a multiple of 16 when parts > 1
    const int mt = m / p.T, t = m - mt * p.T;
    uint4* dst = reinterpret_cast<uint4*>(p.Xq) + ((size_t)mt * chunks) * p.T + t;
    for (int kc = tid; kc < chunks; kc += 256) {
        uint4 q = make_uint4(0u, 0u, 0u, 0u);
        if (kc < live_chunks) {
            const int k0 = kc * 16, part = k0 / pc;
            const int8_t* src = p.codes + ((size_t)part * p.M + m) * pc + (k0 - part * pc);
            if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0 && k0 + 16 <= p.K) {
                q = *reinterpret_cast<const uint4*>(src);
            } else {
                uint32_t w[4] = {0u, 0u, 0u, 0u};
                for (int i = 0; i < 16 && k0 + i < p.K; ++i) w[i >> 2] |= (uint32_t)(uint8_t)src[i] << (8 * (i & 3));
                q = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        dst[(size_t)kc * p.T] = q;
    }
    if (tid == 0) {
        int bad;
        const float s = scale_from_bits(p.rowmax[m], bad);
        p.rowmax[m] = 0u;   // consumed: the next SwiGLU epilogue maxes into a clean word
        p.scales[m] = s;
        p.inverse[m] = __fdiv_rn(1.0f, s);
        // "any row bad" across CTAs: the last CTA to arrive publishes the verdict and clears the scratch
        if (gridDim.x == 1) {
            p.status->bad_input = bad;
        } else {
            if (bad) atomicOr(&p.status->bad_accum, bad);
            __threadfence();
            const unsigned prev = atomicInc(&p.status->done, (unsigned)p.M - 1u);
            if (prev == (unsigned)p.M - 1u) {
                __threadfence();
                p.status->bad_input = atomicExch(&p.status->bad_accum, 0);
            }
        }
    }
}

cudaError_t launch_codes_in(const CodesInParams& p, cudaStream_t stream)
{
    codes_in_kernel<<<(unsigned)p.M, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ reassembly after the all-gather
// One CTA per (row, source rank): the rank's compact row piece goes to its place in the row-major result.
__global__ void __launch_bounds__(128) assemble_columns_kernel(const AssembleParams p)
{
    const int m = blockIdx.x, r = blockIdx.y;
    const int span = p.two_range ? p.N / 2 : p.N;
    int n0, n1;
    shard_range(span, p.world, r, n0, n1);
    const int width = n1 - n0, pieces = p.two_range ? 2 : 1;
    if (width <= 0) return;
    const uint8_t* src_row = p.gathered + (size_t)r * p.slot_bytes + (size_t)m * pieces * width * p.elem;
    for (int piece = 0; piece < pieces; ++piece) {
        const uint8_t* src = src_row + (size_t)piece * width * p.elem;
        uint8_t* dst = p.out + ((size_t)m * p.N + (size_t)piece * span + n0) * p.elem;
        const size_t bytes = (size_t)width * p.elem;
        if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | bytes) & 15u) == 0) {
            for (size_t i = threadIdx.x; i < bytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        } else {
            for (size_t i = threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
        }
    }
}
cudaError_t launch_assemble_columns(const AssembleParams& p, cudaStream_t stream)
{
    if (p.M < 1 || p.world < 1 || p.elem < 1) return cudaErrorInvalidValue;
    assemble_columns_kernel<<<dim3((unsigned)p.M, (unsigned)p.world), 128, 0, stream>>>(p);
    return cudaGetLastError();
}

} // namespace rkb200
