// moe_kernels.cu -- routed SwiGLU experts with int8 weights (the original's rk_npu_moe_w8 operator) for sm_100a.
//
// The original gathers each expert's rows on the NPU, runs int8 GEMMs there and does the middle stage
// (dequantise, SwiGLU, row maximum, nearest-even re-quantisation; src/rk_npu_moe_cpu.cpp:47-115) and the
// weighted combine (src/rk_npu_moe_w8.cpp:786-816) on the CPU.  Here the whole operator is byte work streamed
// from HBM/L2: an expert's weights are read once per job of up to 16 assignments, in records laid out in the
// register order of mma.sync.m16n8k32 so that every warp load is 512 contiguous bytes; the gathered activation
// rows sit in shared memory; sums are exact int32.
//
//   moe_quantize_kernel   fp32 rows -> int8 codes + scales, nearest-even, scale = max/127 (1 for a zero row)
//   moe_gate_up_kernel    per (job, 64 features): gate and up sums of the same feature in the same thread (two warps
//                         per 16 features, half of K each, summed through shared memory),
//                         (float(sum) * s_in) * s_w, y = silu(gate) * up (degree-7 polynomial shared with the dense
//                         path), fp32 middle rows + atomicMax of |y| bit patterns per assignment
//   moe_down_kernel       per (job, 256 columns): re-quantises the job's middle rows into shared memory with the
//                         row scale max/127 (nearest-even), int8 GEMM over I, (float(sum) * s_mid) * s_w
//   moe_combine_kernel    out[token] = sum over the token's slots, in slot order, one fused multiply-add each
#include "moe_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"
#include <algorithm>

namespace rkb200 {

namespace {
constexpr int MOE_FEATURE_BLOCKS = 4;    // gate/up kernel: blocks of 16 features per CTA; two warps share one, half of K each
constexpr int MOE_WARPS = 2 * MOE_FEATURE_BLOCKS;
constexpr int MOE_THREADS = 32 * MOE_WARPS;
constexpr int MOE_DOWN_BLOCKS = 2;       // 16-channel blocks per warp of the down kernel (a CTA covers 256 columns)
constexpr int MOE_ROW_PAD = 16;          // bytes between activation rows in shared memory beyond K: conflict-free fragment loads

__device__ __forceinline__ int8_t nearest_even_code(float v)
{
    return (int8_t)__float2int_rn(fminf(fmaxf(v, -127.f), 127.f));
}

// NB 16-channel blocks (their records at w[0..NB)) against up to 16 activation rows in shared memory:
// c[b][half] += W_b(16 x K) * X^T.  Fragment mapping of m16n8k32 (g = lane / 4, t = lane % 4): A regs = channels g / g + 8
// at k = 4t.. and 16 + 4t..; B regs = token g at the same k; C regs = channels g, g + 8 x tokens 2t, 2t + 1.
// The records of 128 k are double-buffered in registers: while one is multiplied the next is on its way.
// NIB: int4 records (two 16-byte pieces per 128 k instead of four); the sums come out times 16.
template <bool TWO, int NB, bool NIB>
__device__ __forceinline__ void block_mma(const uint4* const (&w)[NB], const uint8_t* xs, int row_bytes, int kq_begin, int kq_count,
                                          int lane, int (&c)[NB][2][4])
{
    constexpr int PIECES = NIB ? 2 : 4;
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* x0 = xs + (size_t)g * row_bytes + 4 * t;
    const uint8_t* x1 = x0 + (size_t)8 * row_bytes;
    uint4 even[NB][PIECES], odd[NB][PIECES];
    auto fetch = [&](uint4 (&a)[NB][PIECES], int kq) {
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int s = 0; s < PIECES; ++s) a[b][s] = __ldg(w[b] + (size_t)(kq * PIECES + s) * 32 + lane);
    };
    auto multiply = [&](const uint4 (&a)[NB][PIECES], int kq) {
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const int k = kq * MOE_KQ + s * 32;
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(x0 + k), b1 = *reinterpret_cast<const uint32_t*>(x0 + k + 16);
            uint32_t d0 = 0, d1 = 0;
            if (TWO) { d0 = *reinterpret_cast<const uint32_t*>(x1 + k); d1 = *reinterpret_cast<const uint32_t*>(x1 + k + 16); }
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                uint32_t a0, a1, a2, a3;
                if (NIB) {
                    const uint4 v = a[b][s >> 1];
                    const uint32_t wx = (s & 1) ? v.z : v.x, wy = (s & 1) ? v.w : v.y;
                    a0 = (wx << 4) & 0xF0F0F0F0u; a2 = wx & 0xF0F0F0F0u;
                    a1 = (wy << 4) & 0xF0F0F0F0u; a3 = wy & 0xF0F0F0F0u;
                } else {
                    const uint4 v = a[b][NIB ? 0 : s];
                    a0 = v.x; a1 = v.y; a2 = v.z; a3 = v.w;
                }
                mma_s8(c[b][0], a0, a1, a2, a3, b0, b1);
                if (TWO) mma_s8(c[b][1], a0, a1, a2, a3, d0, d1);
            }
        }
    };
    if (kq_begin >= kq_count) return;
    fetch(even, kq_begin);
    for (int kq = kq_begin; kq < kq_count; kq += 2) {
        if (kq + 1 < kq_count) fetch(odd, kq + 1);
        multiply(even, kq);
        if (kq + 2 < kq_count) fetch(even, kq + 2);
        if (kq + 1 < kq_count) multiply(odd, kq + 1);
    }
}

// Pulls `bytes` starting at p towards L2, one 128-byte line per lane and step (no data dependence: a hint only).
__device__ __forceinline__ void warp_prefetch_l2(const void* p, size_t bytes, int lane)
{
    const char* c = reinterpret_cast<const char*>(p);
    for (size_t off = (size_t)lane * 128; off < bytes; off += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(c + off));
}
} // namespace

// ------------------------------------------------------------------ weights -> records
__global__ void __launch_bounds__(256) moe_pack_kernel(const MoePackParams p)
{
    const int kq_count = (p.K + MOE_KQ - 1) / MOE_KQ;
    const int pieces = p.nibbles ? 2 : 4;
    const size_t total = (size_t)(p.N / 16) * kq_count * pieces * 32;
    auto code = [&](int k, int n) -> uint32_t { return k < p.K ? (uint32_t)(uint8_t)p.W[(size_t)k * p.N + n] : 0u; };
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int lane = (int)(i & 31), piece = (int)((i >> 5) % pieces);
        const size_t rec = (i >> 5) / pieces;
        const int kq = (int)(rec % kq_count), cb = (int)(rec / kq_count);
        const int g = lane >> 2, t = lane & 3;
        uint32_t word[4];
        if (p.nibbles) {
            // piece = k-steps 2 piece, 2 piece + 1; words: (step, channel g), (step, g + 8), (step + 1, g), (step + 1, g + 8)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int k0 = kq * MOE_KQ + (2 * piece + (r >> 1)) * 32 + 4 * t, n = cb * 16 + g + (r & 1) * 8;
                uint32_t v = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) v |= ((code(k0 + j, n) & 15u) | ((code(k0 + 16 + j, n) & 15u) << 4)) << (8 * j);
                word[r] = v;
            }
        } else {
            const int k0 = kq * MOE_KQ + piece * 32 + 4 * t, n0 = cb * 16 + g;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int k = k0 + (r >> 1) * 16, n = n0 + (r & 1) * 8;
                uint32_t v = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) v |= code(k + j, n) << (8 * j);
                word[r] = v;
            }
        }
        reinterpret_cast<uint4*>(p.packed)[i] = make_uint4(word[0], word[1], word[2], word[3]);
    }
}

// ------------------------------------------------------------------ fp32 rows -> codes (src/rk_npu_moe_w8.cpp:317-343)
__global__ void __launch_bounds__(128) moe_quantize_kernel(const MoeQuantParams p)
{
    __shared__ uint32_t s_max[4];
    __shared__ int s_bad[4];
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = p.X + (size_t)row * p.H;
    uint32_t m = 0;
    int bad = 0;
    for (int i = tid; i < p.H; i += 128) {
        const uint32_t bits = __float_as_uint(x[i]) & 0x7fffffffu;
        bad |= bits >= 0x7f800000u;
        m = max(m, bits);
    }
    m = __reduce_max_sync(0xffffffffu, m);
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) { s_max[warp] = m; s_bad[warp] = bad; }
    __syncthreads();
    m = max(max(s_max[0], s_max[1]), max(s_max[2], s_max[3]));
    bad = s_bad[0] | s_bad[1] | s_bad[2] | s_bad[3];
    const float scale = m ? __fdiv_rn(__uint_as_float(m), 127.f) : 1.f;
    const float inverse = __frcp_rn(scale);
    if (bad || !(scale > 0.f) || (__float_as_uint(inverse) & 0x7fffffffu) >= 0x7f800000u) {
        if (tid == 0) p.status->bad_input = 1;
        return;
    }
    if (tid == 0) p.scales[row] = scale;
    int8_t* q = p.codes + (size_t)row * p.H;
    for (int i = tid; i < p.H; i += 128) q[i] = nearest_even_code(__fmul_rn(x[i], inverse));
}

// ------------------------------------------------------------------ gate/up + SwiGLU
__global__ void __launch_bounds__(MOE_THREADS) moe_gate_up_kernel(const MoeGateUpParams p)
{
    extern __shared__ __align__(16) uint8_t xs[];
    __shared__ float s_scale[MOE_JOB_ROWS];
    __shared__ int s_token[MOE_JOB_ROWS];
    __shared__ int s_partial[MOE_FEATURE_BLOCKS][16][32];
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int job = blockIdx.y;
    // the schedule was uploaded before any kernel of this run started; the weights never change
    const int expert = p.sched.job_expert[job], first = p.sched.job_first[job], rows = p.sched.job_rows[job];
    const int kq_count = (p.H + MOE_KQ - 1) / MOE_KQ;
    const int row_bytes = kq_count * MOE_KQ + MOE_ROW_PAD;
    const int fbi = warp % MOE_FEATURE_BLOCKS, k_half = warp / MOE_FEATURE_BLOCKS;
    const int fb = blockIdx.x * MOE_FEATURE_BLOCKS + fbi;     // block of 16 features
    const bool live = fb * 16 < p.I;
    const int kq_mid = (kq_count + 1) / 2;
    const int kq_begin = k_half ? kq_mid : 0, kq_end = k_half ? kq_count : kq_mid;
    const uint4* base = reinterpret_cast<const uint4*>(p.bank.expert(expert));
    const bool nib = p.bank.nibbles(expert);
    const size_t kq_vecs = nib ? 64 : 128;            // 16-byte pieces of one block per 128 k
    const size_t block_vecs = (size_t)kq_count * kq_vecs;
    const uint4* const w[2] = {base + (size_t)fb * block_vecs, base + (size_t)(p.I / 16 + fb) * block_vecs};
    if (live && kq_end > kq_begin) {
        warp_prefetch_l2(w[0] + (size_t)kq_begin * kq_vecs, (size_t)(kq_end - kq_begin) * kq_vecs * 16, lane);
        warp_prefetch_l2(w[1] + (size_t)kq_begin * kq_vecs, (size_t)(kq_end - kq_begin) * kq_vecs * 16, lane);
    }
    pdl_wait();                                       // fp32 entry: the codes and scales come from the quantise kernel
    if (tid < MOE_JOB_ROWS) {
        const int token = tid < rows ? p.sched.assign_token[first + tid] : -1;
        s_token[tid] = token;
        s_scale[tid] = token >= 0 ? p.in_scales[token] : 0.f;
    }
    __syncthreads();
    // the job's activation rows, 16 bytes per thread and step; rows beyond the job and k beyond H are zero
    {
        const int vec_per_row = row_bytes / 16, h_vec = p.H / 16;   // H is a multiple of 32
        for (int i = tid; i < MOE_JOB_ROWS * vec_per_row; i += MOE_THREADS) {
            const int r = i / vec_per_row, v = i - r * vec_per_row;
            const int token = s_token[r];
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (token >= 0 && v < h_vec) val = *(reinterpret_cast<const uint4*>(p.codes + (size_t)token * p.H) + v);
            *reinterpret_cast<uint4*>(xs + (size_t)r * row_bytes + 16 * v) = val;
        }
    }
    __syncthreads();
    int c[2][2][4] = {};                              // [gate | up][token half][fragment]
    if (live) {
        if (nib) {
            if (rows > 8) block_mma<true, 2, true>(w, xs, row_bytes, kq_begin, kq_end, lane, c);
            else block_mma<false, 2, true>(w, xs, row_bytes, kq_begin, kq_end, lane, c);
        } else {
            if (rows > 8) block_mma<true, 2, false>(w, xs, row_bytes, kq_begin, kq_end, lane, c);
            else block_mma<false, 2, false>(w, xs, row_bytes, kq_begin, kq_end, lane, c);
        }
    }
    // the warp with the upper half of K hands its sums to its partner
    if (k_half == 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) s_partial[fbi][i][lane] = c[i >> 3][(i >> 2) & 1][i & 3];
    }
    __syncthreads();
    if (k_half == 1 || !live) return;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int sum = c[i >> 3][(i >> 2) & 1][i & 3] + s_partial[fbi][i][lane];
        c[i >> 3][(i >> 2) & 1][i & 3] = nib ? sum >> 4 : sum;     // int4 records: every code entered times 16
    }
    const int g = lane >> 2, t = lane & 3;
    const float* ws = p.bank.scales(expert, p.w_scales, 2 * p.I);
    float wg[2], wu[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) { wg[h] = __ldg(ws + fb * 16 + g + 8 * h); wu[h] = __ldg(ws + p.I + fb * 16 + g + 8 * h); }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        if (half == 1 && rows <= 8) break;
        uint32_t mx[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = half * 8 + 2 * t + (i & 1), h = i >> 1;
            if (r < rows) {
                const float sc = s_scale[r];
                const float y = __fmul_rn(silu_poly(dequant(c[0][half][i], sc, wg[h])), dequant(c[1][half][i], sc, wu[h]));
                p.middle[(size_t)(first + r) * p.I + fb * 16 + g + 8 * h] = y;
                mx[i & 1] = max(mx[i & 1], __float_as_uint(y) & 0x7fffffffu);
            }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            uint32_t m = mx[e];
            m = max(m, __shfl_xor_sync(0xffffffffu, m, 4));
            m = max(m, __shfl_xor_sync(0xffffffffu, m, 8));
            m = max(m, __shfl_xor_sync(0xffffffffu, m, 16));
            const int r = half * 8 + 2 * t + e;
            if (g == 0 && r < rows && m) atomicMax(&p.row_max[first + r], m);
        }
    }
}

// ------------------------------------------------------------------ down projection
__global__ void __launch_bounds__(MOE_THREADS) moe_down_kernel(const MoeDownParams p)
{
    extern __shared__ __align__(16) uint8_t xs[];
    __shared__ float s_scale[MOE_JOB_ROWS], s_inverse[MOE_JOB_ROWS];
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int job = blockIdx.y;
    const int expert = p.sched.job_expert[job], first = p.sched.job_first[job], rows = p.sched.job_rows[job];
    const int kq_count = (p.I + MOE_KQ - 1) / MOE_KQ;
    const int row_bytes = kq_count * MOE_KQ + MOE_ROW_PAD;
    const uint4* base = reinterpret_cast<const uint4*>(p.bank.expert(expert));
    const bool nib = p.bank.nibbles(expert);
    const size_t block_vecs = (size_t)kq_count * (nib ? 64 : 128);
    const int cb0 = (blockIdx.x * MOE_WARPS + warp) * MOE_DOWN_BLOCKS;
    {   // this warp's weights on their way to L2 while the gate/up launch still runs
        const int blocks = min(MOE_DOWN_BLOCKS, p.H / 16 - cb0);
        if (blocks > 0) warp_prefetch_l2(base + (size_t)cb0 * block_vecs, (size_t)blocks * block_vecs * 16, lane);
    }
    pdl_wait();                                       // the middle rows and their maxima come from the launch in front
    if (tid < MOE_JOB_ROWS) {
        // src/rk_npu_moe_cpu.cpp:78-80: scale = max/127, 1 for an all-zero row; inverse = 1/scale
        const uint32_t m = tid < rows ? p.row_max[first + tid] : 0u;
        const float scale = m ? __fdiv_rn(__uint_as_float(m), 127.f) : 1.f;
        s_scale[tid] = scale;
        s_inverse[tid] = __frcp_rn(scale);
    }
    __syncthreads();
    {
        const int words_per_row = row_bytes / 4;
        for (int i = tid; i < MOE_JOB_ROWS * words_per_row; i += MOE_THREADS) {
            const int r = i / words_per_row, w = i - r * words_per_row;
            uint32_t packed = 0;
            if (r < rows && 4 * w < p.I) {       // I is a multiple of 32
                const float4 v = *reinterpret_cast<const float4*>(p.middle + (size_t)(first + r) * p.I + 4 * w);
                const float inv = s_inverse[r];
                packed = (uint32_t)(uint8_t)nearest_even_code(__fmul_rn(v.x, inv)) | (uint32_t)(uint8_t)nearest_even_code(__fmul_rn(v.y, inv)) << 8 |
                         (uint32_t)(uint8_t)nearest_even_code(__fmul_rn(v.z, inv)) << 16 | (uint32_t)(uint8_t)nearest_even_code(__fmul_rn(v.w, inv)) << 24;
            }
            *reinterpret_cast<uint32_t*>(xs + (size_t)r * row_bytes + 4 * w) = packed;
        }
    }
    __syncthreads();
    const float* ws = p.bank.scales(expert, p.w_scales, p.H);
    const int g = lane >> 2, t = lane & 3;
#pragma unroll 1
    for (int b = 0; b < MOE_DOWN_BLOCKS; ++b) {
        const int cb = cb0 + b;
        if (cb * 16 >= p.H) break;
        int c[1][2][4] = {};
        const uint4* const w[1] = {base + (size_t)cb * block_vecs};
        if (nib) {
            if (rows > 8) block_mma<true, 1, true>(w, xs, row_bytes, 0, kq_count, lane, c);
            else block_mma<false, 1, true>(w, xs, row_bytes, 0, kq_count, lane, c);
        } else {
            if (rows > 8) block_mma<true, 1, false>(w, xs, row_bytes, 0, kq_count, lane, c);
            else block_mma<false, 1, false>(w, xs, row_bytes, 0, kq_count, lane, c);
        }
        const int shift = nib ? 4 : 0;
        const float w0 = __ldg(ws + cb * 16 + g), w1 = __ldg(ws + cb * 16 + g + 8);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (half == 1 && rows <= 8) break;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = half * 8 + 2 * t + (i & 1), h = i >> 1;
                if (r < rows) p.expert_out[(size_t)(first + r) * p.H + cb * 16 + g + 8 * h] = dequant(c[0][half][i] >> shift, s_scale[r], h ? w1 : w0);
            }
        }
    }
}

// ------------------------------------------------------------------ weighted sum over a token's slots (src/rk_npu_moe_w8.cpp:786-816)
__global__ void __launch_bounds__(256) moe_combine_kernel(const MoeCombineParams p)
{
    pdl_launch_dependents();
    const int token = blockIdx.y;
    const int n = blockIdx.x * 256 + threadIdx.x;
    pdl_wait();
    // the row maxima have been consumed by the down projection: leave them zero for the next run
    if (blockIdx.x == 0 && threadIdx.x < p.slots) {
        const int a = p.slot_assign[token * p.slots + threadIdx.x];
        if (a >= 0) p.row_max[a] = 0u;
    }
    if (n >= p.H) return;
    float sum = 0.f;
    for (int slot = 0; slot < p.slots; ++slot) {
        const int a = p.slot_assign[token * p.slots + slot];
        if (a < 0) continue;
        sum = __fmaf_rn(p.expert_out[(size_t)a * p.H + n], p.coefficients[token * p.slots + slot], sum);
    }
    p.out[(size_t)token * p.H + n] = sum;
}

// ------------------------------------------------------------------ launchers
cudaError_t launch_moe_pack(const MoePackParams& p, cudaStream_t stream)
{
    const size_t total = (p.nibbles ? moe_packed_nibble_bytes(p.K, p.N) : moe_packed_bytes(p.K, p.N)) / 16;
    const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 148 * 8);
    moe_pack_kernel<<<blocks, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_moe_quantize(const MoeQuantParams& p, cudaStream_t stream)
{
    moe_quantize_kernel<<<p.rows, 128, 0, stream>>>(p);
    return cudaGetLastError();
}

static cudaError_t allow_shared(const void* kernel, size_t bytes, PerDeviceOnce& once, size_t& allowed)
{
    int device = -1;
    const bool setup = once.needed(device);
    if (bytes <= 48 * 1024) return cudaSuccess;
    if (setup || bytes > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        allowed = 200 * 1024;
        once.mark(device);
    }
    return bytes <= 200 * 1024 ? cudaSuccess : cudaErrorInvalidValue;
}

// one launch that may start while the kernel in front of it on the stream still runs (each kernel above waits
// with griddepcontrol.wait before it touches what that kernel writes)
template <class Params>
static cudaError_t launch_dependent(void (*kernel)(const Params), dim3 grid, unsigned threads, size_t smem, cudaStream_t stream, const Params& p)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

cudaError_t launch_moe_gate_up(const MoeGateUpParams& p, cudaStream_t stream)
{
    static PerDeviceOnce once;
    static size_t allowed = 0;
    const size_t smem = size_t(MOE_JOB_ROWS) * ((p.H + MOE_KQ - 1) / MOE_KQ * MOE_KQ + MOE_ROW_PAD);
    if (const cudaError_t e = allow_shared(reinterpret_cast<const void*>(moe_gate_up_kernel), smem, once, allowed)) return e;
    const dim3 grid((p.I / 16 + MOE_FEATURE_BLOCKS - 1) / MOE_FEATURE_BLOCKS, p.sched.jobs);
    return launch_dependent(moe_gate_up_kernel, grid, MOE_THREADS, smem, stream, p);
}

cudaError_t launch_moe_down(const MoeDownParams& p, cudaStream_t stream)
{
    const size_t smem = size_t(MOE_JOB_ROWS) * ((p.I + MOE_KQ - 1) / MOE_KQ * MOE_KQ + MOE_ROW_PAD);   // I <= 512: 8.4 KB
    const int per_cta = 16 * MOE_WARPS * MOE_DOWN_BLOCKS;
    const dim3 grid((p.H + per_cta - 1) / per_cta, p.sched.jobs);
    return launch_dependent(moe_down_kernel, grid, MOE_THREADS, smem, stream, p);
}

cudaError_t launch_moe_combine(const MoeCombineParams& p, cudaStream_t stream)
{
    const dim3 grid((p.H + 255) / 256, p.rows);
    return launch_dependent(moe_combine_kernel, grid, 256, 0, stream, p);
}

} // namespace rkb200
