// w4a8_stream.cu -- persistent, evenly balanced tcgen05 W4A8 GEMM for small batches (M <= 32)
// whose weights do not fit on the chip at once (sm_100a).
//
// Why tcgen05 for 1..32 tokens: the legacy mma.sync int8 path of this GPU needs about as long
// for the m16n8k32 instructions of one 8 KB weight block as HBM needs to deliver the block, so
// a weight-streaming kernel built on it is compute-bound from 16 tokens on.  tcgen05.mma
// kind::i8 (M = 128 channels, N = 16 .. 128 tokens) costs a few cycles per block; the only
// per-byte work left is unpacking int4 to int8 into tensor memory, which eight warps do at
// several times the HBM rate.
//
// Schedule: the work is the flat list of (tile of 128 channels, stage of four k-blocks -- two for
// token tiles above 32, whose activation codes take the shared memory --) items, 32 or 16 KB of
// packed weights each, requested as four bulk copies: a thread gets a copy request out only
// every few hundred cycles whatever its size, so requests have to be large -- and every CTA of a persistent grid (one per SM) takes one
// contiguous share of exactly total / CTAs items, so all SMs stream the same number of bytes
// and finish together whatever N and K are.  A CTA's share is a run of segments (tile, stage
// range).  Its copy ring never drains between segments, and the accumulator is double
// buffered in tensor memory, so the epilogue of one segment overlaps the MMAs of the next.
// A segment that covers its tile's whole K is dequantised and stored directly.  Otherwise the
// int32 partial sums are written to a scratch slot of this CTA (a CTA's run begins and ends
// with at most one partial segment each, so it owns two slots) with plain 16-byte stores and
// the tile's stage counter is advanced; whoever brings the counter to the tile's stage count
// works out from the schedule which CTAs contributed, adds their slots (integer addition:
// exact in any order), finishes the tile and leaves the counter zero for the next launch.
// Nobody waits for anybody, and no slot needs clearing.
//
// Roles: warp 0 producer (bulk copies: weights 4 x 8 KB + codes T x 512 B per stage; the first
// ring-full of weights is requested before the programmatic dependency wait), warp 1 MMA
// issuer, warps 2-9 unpack (two sets of four, alternate stages; a stage goes through tensor
// memory as two halves of two k-blocks, each with its own buffer), warps 10-13 epilogue.
// Activation codes and row scales come from quantize_kernel (the launch in front).
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"
#include "w4a8_tc.cuh"

namespace rkb200 {

constexpr int TS_STAGES = 4;
constexpr int TS_KPS_MAX = 4;                // k-blocks per stage: 4 for token tiles up to 32, 2 above (shared memory)
constexpr int TS_ABUF = 7;                   // weight buffers in tensor memory, one half stage (2 k-blocks, 64 columns) each:
                                             // the unpack -> MMA -> commit -> unpack loop is several half-stage times long
constexpr int TS_UNPACK_WARP0 = 2, TS_UNPACK_WARPS = 8;
constexpr int TS_EPI_WARP0 = TS_UNPACK_WARP0 + TS_UNPACK_WARPS, TS_EPI_WARPS = 4;
constexpr int TS_THREADS = 32 * (TS_EPI_WARP0 + TS_EPI_WARPS);   // 448
constexpr int TS_TMEM_COLS = 512;            // two accumulator buffers of max(T, 32) columns, then the weight buffers

__host__ __device__ constexpr int ts_kps(int T) { return T <= 32 ? 4 : 2; }
__host__ __device__ constexpr size_t ts_stage_bytes(int T) { return ts_kps(T) * (8192 + (size_t)T * 128); }
__host__ __device__ constexpr size_t ts_smem_bytes(int T)
{
    return TS_STAGES * ts_stage_bytes(T) + 128 * 4 + (2 * TS_STAGES + 2 * TS_ABUF + 4) * 8 + 32;
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__global__ void __launch_bounds__(TS_THREADS, 1) gemm_tc_stream_kernel(const GemmParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int T = p.T;                                   // 16, 32, 64 or 128 tokens: MMA N, code tile
    const int KPS = ts_kps(T);                           // k-blocks per stage
    const int halves = KPS / 2;                          // a stage passes through tensor memory in pieces of two k-blocks
    const int acc_stride = T < 32 ? 32 : T;              // tensor-memory columns per accumulator buffer
    const int a_col0 = 2 * acc_stride;                   // weight buffers behind the accumulators
    const int abuf = (TS_TMEM_COLS - a_col0) / 64 < TS_ABUF ? (TS_TMEM_COLS - a_col0) / 64 : TS_ABUF;
    const size_t stage_bytes = ts_stage_bytes(T);
    uint8_t* const stages = smem;
    float* const s_sx = reinterpret_cast<float*>(smem + TS_STAGES * stage_bytes);
    uint64_t* const full = reinterpret_cast<uint64_t*>(s_sx + 128);
    uint64_t* const empty = full + TS_STAGES;
    uint64_t* const a_ready = empty + TS_STAGES;
    uint64_t* const a_free = a_ready + TS_ABUF;
    uint64_t* const acc_full = a_free + TS_ABUF;
    uint64_t* const acc_empty = acc_full + 2;
    uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* const s_flag = reinterpret_cast<int*>(s_tmem + 1);   // [0] this CTA completed the tile, [1] a wait ran out

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool swiglu = p.epi == EPI_SWIGLU;
    const int KB = p.KB, KC = KB * 4;
    const int nst = (KB + KPS - 1) / KPS;                // stage iterations per tile
    const int tiles = swiglu ? (p.F + 63) / 64 : (p.N + TILE_N - 1) / TILE_N;
    const long long total = (long long)tiles * nst;
    const long long b0 = total * blockIdx.x / gridDim.x, b1 = total * (blockIdx.x + 1) / gridDim.x;
    const int n_items = (int)(b1 - b0);
    const int tile0 = (int)(b0 / nst), it0 = (int)(b0 - (long long)tile0 * nst);
    const unsigned long long deadline = global_ns() + p.timeout_ns;

    if (tid == 0) {
        for (int s = 0; s < TS_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 5); }   // 4 unpack warps + 1 commit
        for (int b = 0; b < TS_ABUF; ++b) { mbar_init(&a_ready[b], 4); mbar_init(&a_free[b], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], TS_EPI_WARPS); }
        mbar_fence_init();
        s_flag[0] = 0;
        s_flag[1] = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TS_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    // ---------------------------------------------------------------- producer, part 1 (warp 0)
    // (tile, it) advance by counting; lanes 0-3 request one weight group each, lane 4 the codes.
    int pr_tile = tile0, pr_it = it0, pr_gi = 0;
    auto copy_weights = [&](int s, int tile, int it, int kbs) {
        if (lane < 4) {
            const int group = swiglu ? (lane < 2 ? tile * 2 + lane : p.F / GROUP + tile * 2 + (lane - 2)) : tile * 4 + lane;
            bulk_g2s(stages + (size_t)s * stage_bytes + lane * (KPS * 2048), p.Wp + (size_t)group * KC * 512 + (size_t)it * (KPS * 2048), (uint32_t)kbs * 2048u, &full[s]);
        }
    };
    auto copy_codes = [&](int s, int it, int kbs) {
        if (lane == 4) bulk_g2s(stages + (size_t)s * stage_bytes + KPS * 8192, p.Xq + (size_t)it * T * (KPS * 128), (uint32_t)kbs * T * 128u, &full[s]);
    };
    const int pre = n_items < TS_STAGES ? n_items : TS_STAGES;
    if (warp == 0) {
        // Weights never change: the first ring-full is requested before waiting for the kernel in front.
        for (; pr_gi < pre; ++pr_gi) {
            const int kbs = min(KPS, KB - KPS * pr_it);
            if (lane == 0) mbar_expect_tx(&full[pr_gi], (uint32_t)kbs * 8192u);
            __syncwarp();
            copy_weights(pr_gi, pr_tile, pr_it, kbs);
            if (++pr_it == nst) { pr_it = 0; ++pr_tile; }
        }
    }
    pdl_wait();       // activation codes, scales and the status word come from the kernel in front
    const bool skip = *reinterpret_cast<volatile const int*>(&p.status->bad_input) != 0;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer, part 2
        {
            int it = it0;
            for (int gi = 0; gi < pre; ++gi) {
                const int kbs = min(KPS, KB - KPS * it);
                if (lane == 0) { if (skip) mbar_arrive(&full[gi]); else mbar_arrive_expect_tx(&full[gi], (uint32_t)kbs * T * 128u); }
                __syncwarp();
                if (!skip) copy_codes(gi, it, kbs);
                if (++it == nst) it = 0;
            }
        }
        if (skip) {
            // nobody will consume: let the weight copies already requested land before leaving
            if (lane == 0)
                for (int gi = 0; gi < pre; ++gi)
                    if (!mbar_wait(&full[gi], 0, deadline)) { s_flag[1] = 1; break; }
        } else {
            for (; pr_gi < n_items; ++pr_gi) {
                const int s = pr_gi % TS_STAGES;
                const int kbs = min(KPS, KB - KPS * pr_it);
                int ok = 1;
                if (lane == 0) {
                    ok = mbar_wait(&empty[s], ((pr_gi / TS_STAGES) - 1) & 1, deadline) ? 1 : 0;
                    if (ok) mbar_arrive_expect_tx(&full[s], (uint32_t)kbs * (8192u + T * 128u));
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { s_flag[1] = 1; break; }
                copy_weights(s, pr_tile, pr_it, kbs);
                copy_codes(s, pr_it, kbs);
                if (++pr_it == nst) { pr_it = 0; ++pr_tile; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0 && !skip) {
            const uint32_t idesc = tc_idesc_s8(128, T);
            bool ok = true;
            int gi = 0, seg = 0, tile = tile0, it = it0;
            while (gi < n_items && ok) {
                const int nseg = min(nst - it, n_items - gi);
                const int buf = seg & 1;
                if (seg >= 2) {   // the epilogue has read this accumulator buffer's previous segment
                    ok = mbar_wait(&acc_empty[buf], ((seg >> 1) - 1) & 1, deadline);
                    if (!ok) { s_flag[1] = 1; break; }
                    tc_fence_after();
                }
                const uint32_t d_tmem = tmem_base + buf * acc_stride;
                for (int i = 0; i < nseg && ok; ++i) {
                    const int g = gi + i, s = g % TS_STAGES;
                    const int kbs = min(KPS, KB - KPS * (it + i));
                    const uint32_t xaddr = smem_u32(stages + (size_t)s * stage_bytes + KPS * 8192);
                    for (int half = 0; half < halves && ok; ++half) {
                        const int h = halves * g + half, b = h % abuf;
                        const int kh = min(2, kbs - 2 * half);           // k-blocks in this half (<= 0: none, bookkeeping only)
                        ok = mbar_wait(&a_ready[b], (h / abuf) & 1, deadline);
                        if (!ok) { s_flag[1] = 1; break; }
                        tc_fence_after();
                        const uint32_t a_tmem = tmem_base + a_col0 + b * 64;
                        // k-step q of the half: k-block q / 4, 32 k = two 16-byte chunks per token, i.e. the
                        // descriptor's address field advances by 2 * T (16-byte units) per step
                        const uint64_t desc0 = tc_smem_desc(xaddr + (uint32_t)(2 * half) * T * 128, (uint32_t)T * 16u, 128u);
                        const uint64_t step = (uint64_t)(2 * T);
                        if (kh >= 1) {
                            tc_mma_i8_ts(d_tmem, a_tmem, desc0, idesc, (i > 0 || half > 0) ? 1u : 0u);
#pragma unroll
                            for (int q = 1; q < 4; ++q) tc_mma_i8_ts_acc(d_tmem, a_tmem + q * 8, desc0 + q * step, idesc);
                        }
                        if (kh >= 2) {
#pragma unroll
                            for (int q = 4; q < 8; ++q) tc_mma_i8_ts_acc(d_tmem, a_tmem + q * 8, desc0 + q * step, idesc);
                        }
                        tc_commit(&a_free[b]);   // the weight buffer may be rewritten once these MMAs retire
                    }
                    if (ok) tc_commit(&empty[s]);   // and the stage refilled
                }
                if (!ok) break;
                tc_commit(&acc_full[buf]);
                gi += nseg;
                it += nseg;
                if (it == nst) { it = 0; ++tile; }
                ++seg;
            }
            (void)tile;
        }
    } else if (warp < TS_EPI_WARP0) {
        // ---------------------------------------------------------------- weight unpack -> TMEM
        const int q = warp & 3;
        const int set = (warp - TS_UNPACK_WARP0) >> 2;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        // plain: group q, row lane.  SwiGLU: lanes 0-15 gate rows, lanes 16-31 the matching up
        // rows (staged groups 0,1 = gate, 2,3 = up of the same 64 features).
        const int src_group = swiglu ? (q >> 1) + (lane >= 16 ? 2 : 0) : q;
        const int src_row = swiglu ? (q & 1) * 16 + (lane & 15) : lane;
        bool ok = !skip;
        int it = it0;
        for (int g = 0; g < n_items && ok; ++g) {
            const int kbs = min(KPS, KB - KPS * it);
            if (++it == nst) it = 0;
            if ((g & 1) != set) continue;                      // the two sets take alternate stages
            const int s = g % TS_STAGES;
            ok = mbar_wait(&full[s], (g / TS_STAGES) & 1, deadline);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { s_flag[1] = 1; break; }
            for (int half = 0; half < halves && ok; ++half) {
                const int h = halves * g + half, b = h % abuf;
                const int kh = min(2, kbs - 2 * half);           // k-blocks in this half (<= 0: none, bookkeeping only)
                if (h >= abuf) ok = mbar_wait(&a_free[b], ((h / abuf) - 1) & 1, deadline);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { s_flag[1] = 1; break; }
                tc_fence_after();
                const uint4* src = reinterpret_cast<const uint4*>(stages + (size_t)s * stage_bytes + src_group * (KPS * 2048) + half * 4096) + src_row;
                uint4 w[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) w[c] = (c < 4 * kh) ? src[c * 32] : make_uint4(0u, 0u, 0u, 0u);
                if (half == halves - 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[s]);   // the packed copy is in registers; the codes stay until the commit
                }
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    if (hh < kh) {
                        uint32_t r[32];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t ww[4] = {w[4 * hh + c].x, w[4 * hh + c].y, w[4 * hh + c].z, w[4 * hh + c].w};
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) {
                                r[c * 8 + jj] = (ww[jj] << 4) & 0xF0F0F0F0u;
                                r[c * 8 + 4 + jj] = ww[jj] & 0xF0F0F0F0u;
                            }
                        }
                        tc_st32(lane_addr + a_col0 + b * 64 + hh * 32, r);
                    }
                }
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_ready[b]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps
        const int q = warp & 3;                        // TMEM lane quarter this warp may read
        const int et = tid - 32 * TS_EPI_WARP0;        // 0..127 among the epilogue threads
        const int row = q * 32 + lane;                 // accumulator row (TMEM lane) of this thread
        const int out_cols = swiglu ? p.F : p.N;
        // output column inside the tile this row belongs to
        const int col = swiglu ? (q >> 1) * 32 + (q & 1) * 16 + (lane & 15) : row;
        const bool up_lane = swiglu && lane >= 16;
        bool ok = !skip;
        int gi = 0, seg = 0, tile = tile0, it = it0;
        s_sx[et] = et < p.M ? p.sx[et] : 0.f;   // visible to all four warps after the first barrier below
        const int nchunk = (T + 31) / 32;        // the accumulator is read in pieces of up to 32 token columns
        // finish 32 tokens of one output channel: dequantise (+ SwiGLU), store
        auto finish_chunk = [&](const int (&v)[32], int tile, int c) {
            const int n = (swiglu ? tile * 64 : tile * TILE_N) + col;
            const bool n_ok = n < out_cols;
            const float sw = n_ok ? p.sw[(up_lane ? p.F : 0) + n] : 0.f;
            const int m0 = 32 * c;
            float y[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) y[i] = dequant(v[i], s_sx[m0 + i], sw);
            if (p.epi == EPI_F16) {
                __half* const out = reinterpret_cast<__half*>(p.out) + (size_t)m0 * out_cols + n;
                if (n_ok) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (m0 + i < p.M) out[(size_t)i * out_cols] = __float2half_rn(y[i]);
                }
            } else if (p.epi == EPI_F32) {
                float* const out = reinterpret_cast<float*>(p.out) + (size_t)m0 * out_cols + n;
                if (n_ok) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (m0 + i < p.M) out[(size_t)i * out_cols] = y[i];
                }
            } else if (p.epi == EPI_I32) {
                int* const out = reinterpret_cast<int*>(p.out) + (size_t)m0 * out_cols + n;
                if (n_ok) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (m0 + i < p.M) out[(size_t)i * out_cols] = v[i];
                }
            } else {
                uint32_t mx[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float up = __shfl_xor_sync(0xffffffffu, y[i], 16);       // gate lanes receive u
                    y[i] = __fmul_rn(silu_poly(y[i]), up);                          // meaningful in gate lanes
                    const bool live = !up_lane && n_ok && m0 + i < p.M;
                    mx[i] = live ? (__float_as_uint(y[i]) & 0x7fffffffu) : 0u;
                }
                if (p.rowmax) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx[i] = __reduce_max_sync(0xffffffffu, mx[i]);
                }
                float* const out = reinterpret_cast<float*>(p.out) + (size_t)m0 * out_cols + n;
                if (!up_lane && n_ok) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (m0 + i < p.M) out[(size_t)i * out_cols] = y[i];
                }
                if (p.rowmax && lane == 0) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (m0 + i < p.M && mx[i]) atomicMax(&p.rowmax[m0 + i], mx[i]);
                }
            }
        };
        while (gi < n_items && ok) {
            const int nseg = min(nst - it, n_items - gi);
            const int buf = seg & 1;
            ok = mbar_wait(&acc_full[buf], (seg >> 1) & 1, deadline);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { s_flag[1] = 1; }
            // All four warps take the same decision after the next barrier.
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (*reinterpret_cast<volatile int*>(&s_flag[1])) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * acc_stride;
            const bool whole = nseg == nst;          // this segment covers its tile's whole K
            // slot layout [token / 4][row][4 tokens]: a warp's 16-byte accesses are contiguous
            int4* const scratch = reinterpret_cast<int4*>(p.partials);
            int4* const my_slot = scratch + (size_t)(2 * blockIdx.x + (gi == 0 ? 0 : 1)) * 32 * T;
            for (int c = 0; c < nchunk; ++c) {
                uint32_t r[32];
                tc_ld16(taddr + 32 * c, r);
                if (T > 16) tc_ld16(taddr + 32 * c + 16, r + 16);
                else {
#pragma unroll
                    for (int i = 16; i < 32; ++i) r[i] = 0u;
                }
                tc_wait_ld();
                if (c == nchunk - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_relaxed(&acc_empty[buf]);   // the MMAs of segment seg + 2 may overwrite it
                }
                int v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = (int)r[i] >> 4;     // exact: sums are multiples of 16
                if (whole) finish_chunk(v, tile, c);
                else {
                    // ---- part of a tile: into this CTA's slot
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (32 * c + 4 * j < T)
                            my_slot[(size_t)(8 * c + j) * 128 + row] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
            if (!whole) {
                // ---- advance the tile's stage counter; whoever completes it finishes the tile
                __threadfence();
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (et == 0) {
                    const unsigned before = atomicAdd(p.counts + tile, (unsigned)nseg);
                    s_flag[0] = (before + (unsigned)nseg == (unsigned)nst) ? 1 : 0;
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                const bool finish = *reinterpret_cast<volatile int*>(&s_flag[0]) != 0;
                if (finish) {
                    // last contributor: every CTA whose share of the flat list overlaps this tile's stages wrote a
                    // slot -- its first one if its run starts in this tile, else its second
                    __threadfence();
                    const long long s0 = (long long)tile * nst, s1 = s0 + nst, grid = gridDim.x;
                    int c_lo = (int)(s0 * grid / total);
                    while (total * (c_lo + 1) / grid <= s0) ++c_lo;
                    while (total * c_lo / grid > s0) --c_lo;
                    for (int c = 0; c < nchunk; ++c) {
                        int v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0;
                        for (int cc = c_lo; cc < (int)grid && total * cc / grid < s1; ++cc) {
                            const int first_tile = (int)((total * cc / grid) / nst);
                            const int4* const src = scratch + (size_t)(2 * cc + (first_tile == tile ? 0 : 1)) * 32 * T;
                            int4 part[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                part[j] = (32 * c + 4 * j < T) ? __ldcg(src + (size_t)(8 * c + j) * 128 + row) : make_int4(0, 0, 0, 0);
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                v[4 * j] += part[j].x; v[4 * j + 1] += part[j].y; v[4 * j + 2] += part[j].z; v[4 * j + 3] += part[j].w;
                            }
                        }
                        finish_chunk(v, tile, c);
                    }
                    if (et == 0) p.counts[tile] = 0u;
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");   // s_flag[0] may be rewritten by the next segment
            }
            gi += nseg;
            it += nseg;
            if (it == nst) { it = 0; ++tile; }
            ++seg;
        }
    }

    // ------------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && s_flag[1]) atomicExch(&p.status->device_error, 1);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TS_TMEM_COLS) : "memory");
    }
}

cudaError_t launch_gemm_stream(const GemmParams& p, int sm_count, cudaStream_t stream, bool pdl)
{
    if ((p.T != 16 && p.T != 32 && p.T != 64 && p.T != 128) || p.M > p.T || (long long)p.KB * KBLOCK > 131072 || !p.partials || !p.counts)
        return cudaErrorInvalidValue;
    static PerDeviceOnce configured;
    int configured_device = -1;
    if (configured.needed(configured_device)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ts_smem_bytes(128) > ts_smem_bytes(32) ? ts_smem_bytes(128) : ts_smem_bytes(32)));
        if (e != cudaSuccess) return e;
        configured.mark(configured_device);
    }
    const int tiles = p.epi == EPI_SWIGLU ? (p.F + 63) / 64 : (p.N + TILE_N - 1) / TILE_N;
    const long long total = (long long)tiles * ((p.KB + ts_kps(p.T) - 1) / ts_kps(p.T));
    long long ctas = sm_count;
    if (ctas > total / 2) ctas = total / 2 > 0 ? total / 2 : 1;   // at least two stages per CTA
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(TS_THREADS);
    cfg.dynamicSmemBytes = ts_smem_bytes(p.T);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemm_tc_stream_kernel, p);
}

} // namespace rkb200
