// w4a8_gemm_tc.cu -- tcgen05 W4A8 GEMM for large batches (prefill) on sm_100a.
//
// Replaces the reference's device step plus its CPU reconstruction: the INT4 x INT4 ->
// INT16 partial products of src/rk_npu_i4_regs.cpp:7-51, the split-K INT16 -> INT32
// accumulation and the dequantising / SwiGLU epilogues of src/rk_npu_w4a8_output.cpp:35-161
// and src/rk_npu_w4a8_swiglu.cpp:12-91 become one kernel with exact int32 accumulation.
//
// Swap-AB mapping: the 128 output channels of a CTA are the M side of tcgen05.mma
// (kind::i8, M = 128), the tokens of one tile (T <= 256) the N side, accumulators int32 in
// tensor memory.  Per 128-element k-block:
//   warp 0      one thread streams the packed int4 weights (4 x 2 KB) and the int8
//               activation tile (T x 128 B) with bulk async copies into a ring of stages;
//   warps 2-9   unpack the int4 weights (three ALU instructions per eight codes) and write
//               them with tcgen05.st into a ring of TMEM buffers: the MMA's A operand comes
//               from tensor memory, so unpacked weights never touch shared memory.  Two sets
//               of four warps (one warp per TMEM lane quarter) take alternate k-blocks, and a
//               warp overlaps the store of one k-block with the unpacking of its next;
//   warp 1      one thread issues four tcgen05.mma (K = 32 each) with the activation tile as
//               shared-memory B operand (K-major, no swizzle: the tile already is a sequence
//               of 8 x 16-byte core matrices) and commits the stage / buffer back.
// Warps 2-9 then read the accumulators with tcgen05.ld and run the epilogue.
// Every wait is bounded by the workspace's timeout; a wait that runs out sets the status
// word, the kernel drains and frees its tensor memory and returns.
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"

namespace rkb200 {

constexpr int TC_STAGES = 5;
constexpr int TC_ABUF = 8;
constexpr int TC_UNPACK_WARPS = 8;   // two sets of four (one warp per TMEM lane quarter), alternating k-blocks
constexpr int TC_THREADS = 64 + 32 * TC_UNPACK_WARPS;
constexpr int TC_A_COL0 = 256;      // A buffers live behind the accumulator columns
constexpr int TC_TMEM_COLS = 512;

__host__ __device__ constexpr size_t tc_stage_bytes(int T) { return 8192 + (size_t)T * 128; }
__host__ __device__ constexpr size_t tc_smem_bytes(int T)
{
    return TC_STAGES * tc_stage_bytes(T) + (size_t)T * 4 /* token scales */ + (2 * TC_STAGES + 2 * TC_ABUF + 1) * 8 + 32;
}

// ---- tcgen05 wrappers
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major, no swizzle.  A core matrix is eight rows of
// 16 bytes, contiguous (128 B); `lbo` = bytes between core matrices adjacent in K, `sbo` =
// bytes between core matrices adjacent in the row (token) direction.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo)
{
    const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16);
    const uint32_t hi = (sbo >> 4) | (1u << 14);   // descriptor version 1 (sm_100); layout type 0 = no swizzle
    return ((uint64_t)hi << 32) | lo;
}
// Instruction descriptor: int32 accumulators, signed 8-bit A and B, both K-major, M = 128.
__device__ __forceinline__ uint32_t tc_idesc_s8(int n)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const GemmParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int T = p.T;
    const size_t stage_bytes = tc_stage_bytes(T);
    uint8_t* const stages = smem;
    float* const s_sx = reinterpret_cast<float*>(smem + TC_STAGES * stage_bytes);
    uint64_t* const full = reinterpret_cast<uint64_t*>(s_sx + T);
    uint64_t* const empty = full + TC_STAGES;
    uint64_t* const a_ready = empty + TC_STAGES;
    uint64_t* const a_free = a_ready + TC_ABUF;
    uint64_t* const acc_done = a_free + TC_ABUF;
    uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(acc_done + 1);
    int* const s_error = reinterpret_cast<int*>(s_tmem + 1);

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, mt = blockIdx.y;
    const bool swiglu = p.epi == EPI_SWIGLU;
    const int KB = p.KB, KC = KB * 4;
    const unsigned long long deadline = global_ns() + p.timeout_ns;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 5); }
        for (int b = 0; b < TC_ABUF; ++b) { mbar_init(&a_ready[b], 4); mbar_init(&a_free[b], 1); }
        mbar_init(acc_done, 1);
        mbar_fence_init();
        *s_error = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    pdl_wait();   // activation codes, scales and the status word come from the kernel in front
    const bool skip = *reinterpret_cast<volatile const int*>(&p.status->bad_input) != 0;

    if (!skip) {
        if (warp == 0) {
            // ---------------------------------------------------------------- producer
            if (lane == 0) {
                int group[4];
#pragma unroll
                for (int w = 0; w < 4; ++w)
                    group[w] = swiglu ? (w < 2 ? tile * 2 + w : p.F / GROUP + tile * 2 + (w - 2)) : tile * 4 + w;
                const uint8_t* xtile = p.Xq + (size_t)mt * ((size_t)KB * 8) * T * 16;
                for (int kb = 0; kb < KB; ++kb) {
                    const int s = kb % TC_STAGES;
                    if (kb >= TC_STAGES && !mbar_wait(&empty[s], ((kb / TC_STAGES) - 1) & 1, deadline)) { *s_error = 1; break; }
                    uint8_t* dst = stages + (size_t)s * stage_bytes;
                    mbar_arrive_expect_tx(&full[s], (uint32_t)stage_bytes);
#pragma unroll
                    for (int w = 0; w < 4; ++w)
                        bulk_g2s(dst + w * 2048, p.Wp + ((size_t)group[w] * KC + (size_t)kb * 4) * 512, 2048, &full[s]);
                    bulk_g2s(dst + 8192, xtile + (size_t)kb * 8 * T * 16, (uint32_t)T * 128u, &full[s]);
                }
            }
        } else if (warp == 1) {
            // ---------------------------------------------------------------- MMA issuer
            if (lane == 0) {
                const uint32_t idesc = tc_idesc_s8(T);
                bool ok = true;
                for (int kb = 0; kb < KB && ok; ++kb) {
                    const int s = kb % TC_STAGES, b = kb % TC_ABUF;
                    ok = mbar_wait(&full[s], (kb / TC_STAGES) & 1, deadline) && mbar_wait(&a_ready[b], (kb / TC_ABUF) & 1, deadline);
                    if (!ok) { *s_error = 1; break; }
                    tc_fence_after();
                    const uint32_t xaddr = smem_u32(stages + (size_t)s * stage_bytes + 8192);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t desc = tc_smem_desc(xaddr + (uint32_t)(2 * j) * T * 16, (uint32_t)T * 16u, 128u);
                        tc_mma_i8_ts(tmem_base, tmem_base + TC_A_COL0 + b * 32 + j * 8, desc, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    }
                    tc_commit(&empty[s]);    // activation stage may be refilled once these MMAs retire
                    tc_commit(&a_free[b]);   // and the weight buffer in tensor memory rewritten
                }
                tc_commit(acc_done);
            }
        } else {
            // ---------------------------------------------------------------- weight unpack -> TMEM
            const int q = warp & 3;                       // TMEM lane quarter == weight group of the tile
            const int set = (warp - 2) >> 2;              // this set takes k-blocks kb % 2 == set
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            bool ok = true;
            int pending = -1;                             // buffer whose tensor-memory store is in flight
            for (int kb = set; kb < KB && ok; kb += 2) {
                const int s = kb % TC_STAGES, b = kb % TC_ABUF;
                ok = mbar_wait(&full[s], (kb / TC_STAGES) & 1, deadline);
                if (ok && kb >= TC_ABUF) ok = mbar_wait(&a_free[b], ((kb / TC_ABUF) - 1) & 1, deadline);
                ok = __all_sync(0xffffffffu, ok);   // the tensor-memory store below needs the whole warp
                if (!ok) { *s_error = 1; break; }
                tc_fence_after();
                const uint4* src = reinterpret_cast<const uint4*>(stages + (size_t)s * stage_bytes + q * 2048) + lane;
                uint32_t r[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 w = src[c * 32];
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        r[c * 8 + j] = (ww[j] << 4) & 0xF0F0F0F0u;       // k = 32c + 4j .. +3      (x16)
                        r[c * 8 + 4 + j] = ww[j] & 0xF0F0F0F0u;          // k = 32c + 16 + 4j .. +3 (x16)
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);    // the packed weights of this stage are in registers
                if (pending >= 0) {                        // the previous store had the unpacking above to complete
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_ready[pending]);
                }
                tc_st32(lane_addr + TC_A_COL0 + b * 32, r);
                pending = b;
            }
            if (pending >= 0) {
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_ready[pending]);
            }
        }

        // -------------------------------------------------------------------- epilogue
        if (warp >= 2) {
            const int q = warp & 3;
            const int set = (warp - 2) >> 2;              // the two sets take alternate 32-token chunks
            for (int i = tid - 64; i < T; i += 32 * TC_UNPACK_WARPS) {
                const int m = mt * T + i;
                s_sx[i] = m < p.M ? p.sx[m] : 0.f;
            }
            if (!mbar_wait(acc_done, 0, deadline)) *s_error = 1;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const bool done = *reinterpret_cast<volatile int*>(s_error) == 0;   // same answer in all 128 threads
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            float* const exch = reinterpret_cast<float*>(stages) + set * 2048;   // all stages are drained by now
            const int ch = q * 32 + lane;
            int n;                                        // global output channel of this thread
            if (swiglu) n = ch < 64 ? tile * 64 + ch : p.F + tile * 64 + (ch - 64);
            else n = tile * TILE_N + ch;
            const bool n_ok = swiglu ? (tile * 64 + (ch & 63)) < p.F : n < p.N;
            const float sw = n_ok ? p.sw[n] : 0.f;
            for (int t0 = set * 32; t0 < T && done; t0 += 64) {
                uint32_t r[32];
                tc_ld32(lane_addr + t0, r);
                tc_wait_ld();
                if (!swiglu) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int m = mt * T + t0 + i;
                        if (t0 + i < T && m < p.M && n_ok) {
                            const int v = (int)r[i] >> 4;   // exact: sums are multiples of 16
                            if (p.epi == EPI_I32) reinterpret_cast<int*>(p.out)[(size_t)m * p.N + n] = v;
                            else {
                                const float y = dequant(v, s_sx[t0 + i], sw);
                                if (p.epi == EPI_F32) reinterpret_cast<float*>(p.out)[(size_t)m * p.N + n] = y;
                                else reinterpret_cast<__half*>(p.out)[(size_t)m * p.N + n] = __float2half_rn(y);
                            }
                        }
                    }
                } else {
                    // lanes 64..127 of the accumulator hold the up projection of the same 64
                    // features: hand it to the gate threads through shared memory
                    if (ch >= 64) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            exch[i * 64 + (ch - 64)] = dequant((int)r[i] >> 4, t0 + i < T ? s_sx[t0 + i] : 0.f, sw);
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + set) : "memory");
                    if (ch < 64) {
                        const int f = tile * 64 + ch;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int m = mt * T + t0 + i;
                            const float g = dequant((int)r[i] >> 4, t0 + i < T ? s_sx[t0 + i] : 0.f, sw);
                            const float y = __fmul_rn(silu_poly(g), exch[i * 64 + ch]);
                            const bool ok = t0 + i < T && m < p.M && n_ok;
                            if (ok) reinterpret_cast<float*>(p.out)[(size_t)m * p.F + f] = y;
                            if (p.rowmax) {
                                const uint32_t mx = __reduce_max_sync(0xffffffffu, ok ? (__float_as_uint(y) & 0x7fffffffu) : 0u);
                                if (lane == 0 && mx) atomicMax(&p.rowmax[m], mx);
                            }
                        }
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + set) : "memory");
                }
            }
        }
    }

    // ------------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *s_error) atomicExch(&p.status->device_error, 1);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

bool gemm_tc_supported(const GemmParams& p)
{
    // 16 x |sum| must fit int32 (see the packed-weight layout), and the kernel keeps all of K in one CTA.
    return p.M >= 1 && (long long)p.KB * KBLOCK <= 131072;
}

cudaError_t launch_gemm_tc(const GemmParams& p, cudaStream_t stream, bool pdl)
{
    if (p.T < 16 || p.T > 256 || p.T % 16 || !gemm_tc_supported(p)) return cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(256));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int tiles = p.epi == EPI_SWIGLU ? (p.F + 63) / 64 : p.NG / 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles, (unsigned)((p.M + p.T - 1) / p.T), 1);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = tc_smem_bytes(p.T);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel, p);
}

} // namespace rkb200
