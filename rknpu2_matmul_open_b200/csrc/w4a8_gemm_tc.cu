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
//
// Two forms share the code.  PAIR = false: one CTA, token tile T <= 256 (batches of 33..128
// tokens).  PAIR = true: two CTAs of a cluster form one 256-channel x 256-token tile with
// tcgen05.mma.cta_group::2: each CTA unpacks its own 128 channels into its own tensor memory
// and loads only its half (128 tokens) of the activation tile, which halves the activation
// traffic per MMA; the leader CTA issues the MMAs for both and signals both with multicast
// commits.  The activation loads stay plain (non-multicast) bulk copies.
// Every wait is bounded by the workspace's timeout; a wait that runs out sets the status
// word, the kernel drains and frees its tensor memory and returns.
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"
#include "w4a8_tc.cuh"

namespace rkb200 {

// A stage holds TWO k-blocks, so five bulk copies feed two k-blocks of MMAs (the copy engine
// sustains only a few requests in flight per SM; fewer, larger requests keep it ahead).
constexpr int TC_STAGES = 2;          // single-CTA form, T > 128: 2 x (8 KB weights + T x 128 B activations) per stage
constexpr int TC_STAGES_DEEP = 4;     // single-CTA form, T <= 128: the copies take several stage times to arrive
constexpr int TC_STAGES_PAIR = 4;     // paired form: 2 x (8 KB + 16 KB) per stage
constexpr int TC_ABUF = 8;
constexpr int TC_UNPACK_WARPS = 8;   // two sets of four (one warp per TMEM lane quarter), alternating k-blocks
constexpr int TC_THREADS = 64 + 32 * TC_UNPACK_WARPS;
constexpr int TC_A_COL0 = 256;      // A buffers live behind the accumulator columns
constexpr int TC_TMEM_COLS = 512;

// bytes of one k-block of one 32-channel weight group: int4 codes 2 KB, int8 codes (the W8A8 operators) 4 KB
__host__ __device__ constexpr size_t tc_group_bytes(bool w8) { return w8 ? 4096 : 2048; }
__host__ __device__ constexpr size_t tc_stage_bytes(int T, bool w8 = false) { return 2 * (4 * tc_group_bytes(w8) + (size_t)T * 128); }
__host__ __device__ constexpr size_t tc_smem_bytes(int T, int stages, int tokens, bool w8 = false)
{
    return stages * tc_stage_bytes(T, w8) + (size_t)tokens * 4 /* token scales */ + (2 * stages + 2 * TC_ABUF + 1) * 8 + 32;
}
// Ring depth of a form: the depth the int4 form was tuned with, fewer where int8 weights (twice the bytes) would not fit
__host__ __device__ constexpr int tc_stage_count(int T, bool pair, bool w8)
{
    int stages = pair ? TC_STAGES_PAIR : (T <= 128 ? TC_STAGES_DEEP : TC_STAGES);
    while (stages > 2 && tc_smem_bytes(T, stages, pair ? 256 : T, w8) > 225 * 1024) --stages;
    return stages;
}

template <bool PAIR, bool W8>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const GemmParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int NSTAGE = tc_stage_count(p.T, PAIR, W8);
    const int T = p.T;                              // tokens of this CTA's activation tile (128 when paired)
    const int TOK = PAIR ? 256 : T;                 // tokens (accumulator columns) of the MMA tile
    const size_t stage_bytes = tc_stage_bytes(T, W8);
    constexpr uint32_t GB = (uint32_t)tc_group_bytes(W8);   // one k-block of one weight group
    uint8_t* const stages = smem;
    float* const s_sx = reinterpret_cast<float*>(smem + NSTAGE * stage_bytes);
    uint64_t* const full = reinterpret_cast<uint64_t*>(s_sx + TOK);
    uint64_t* const empty = full + NSTAGE;
    uint64_t* const a_ready = empty + NSTAGE;
    uint64_t* const a_free = a_ready + TC_ABUF;
    uint64_t* const acc_done = a_free + TC_ABUF;
    uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(acc_done + 1);
    int* const s_error = reinterpret_cast<int*>(s_tmem + 1);

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x;
    const uint32_t rank = PAIR ? cluster_rank() : 0u;          // 0 = leader of the pair
    const int mt = PAIR ? 2 * (int)blockIdx.y + (int)rank : (int)blockIdx.y;   // this CTA's activation tile
    const int tok_base = (int)blockIdx.y * TOK;                 // first token of the MMA tile
    const bool swiglu = p.epi == EPI_SWIGLU;
    const int KB = p.KB, KC = KB * 4;
    const unsigned long long deadline = global_ns() + p.timeout_ns;
    unsigned long long* const trace = (p.trace && blockIdx.x < 2 && blockIdx.y == 0) ? p.trace + blockIdx.x * 1024 : nullptr;
    const long long c0 = clock64();
    if (trace && threadIdx.x == 0) trace[770] = global_ns();
#define TC_STAMP(role, kb, slot) do { if (trace && (kb) < 64) trace[((role) * 64 + (kb)) * 4 + (slot)] = (unsigned long long)(clock64() - c0); } while (0)

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 5); }   // 4 unpack warps + 1 commit
        for (int b = 0; b < TC_ABUF; ++b) { mbar_init(&a_ready[b], PAIR ? 8 : 4); mbar_init(&a_free[b], 1); }
        mbar_init(acc_done, 1);
        mbar_fence_init();
        *s_error = 0;
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TC_TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TC_TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) { cluster_arrive(); cluster_wait(); }   // the peer's barriers and tensor memory exist from here on
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    pdl_wait();   // activation codes, scales and the status word come from the kernel in front
    const bool skip = *reinterpret_cast<volatile const int*>(&p.status->bad_input) != 0;

    if (!skip) {
        if (warp == 0) {
            // ---------------------------------------------------------------- producer
            // Lane 0 waits for the stage and arms its barrier; lanes 0-3 then each request one
            // weight group and lane 4 the activation tile, so the five requests issue in parallel.
            const int w = lane & 3;
            const int group = swiglu ? (w < 2 ? tile * 2 + w : p.F / GROUP + tile * 2 + (w - 2)) : tile * 4 + w;
            const uint8_t* wsrc = p.Wp + (size_t)group * KB * GB;
            const uint8_t* xtile = p.Xq + (size_t)mt * ((size_t)KB * 8) * T * 16;
            bool ok = true;
            const int nstage_iters = (KB + 1) / 2;
            for (int it = 0; it < nstage_iters && ok; ++it) {
                const int s = it % NSTAGE;
                const int kbs = min(2, KB - 2 * it);              // k-blocks in this stage
                if (lane == 0) {
                    if (it >= NSTAGE) ok = mbar_wait_cluster(&empty[s], ((it / NSTAGE) - 1) & 1, deadline);
                    if (ok) mbar_arrive_expect_tx(&full[s], (uint32_t)kbs * (4u * GB + (uint32_t)T * 128u));
                    TC_STAMP(0, 2 * it, 0);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { *s_error = 1; break; }
                uint8_t* dst = stages + (size_t)s * stage_bytes;
                if (lane < 4) bulk_g2s(dst + w * 2 * GB, wsrc + (size_t)it * 2 * GB, (uint32_t)kbs * GB, &full[s]);
                else if (lane == 4) bulk_g2s(dst + 8 * GB, xtile + (size_t)it * 16 * T * 16, (uint32_t)kbs * (uint32_t)T * 128u, &full[s]);
            }
        } else if (warp == 1) {
            // ---------------------------------------------------------------- MMA issuer
            // (paired form: the leader issues for both CTAs; a_ready counts the unpack warps of
            // both, each of which has seen its own stage complete, activation half included)
            if (lane == 0 && rank == 0) {
                const uint32_t idesc = tc_idesc_s8(PAIR ? 256 : 128, TOK);
                bool ok = true;
                for (int kb = 0; kb < KB && ok; ++kb) {
                    const int it = kb >> 1, s = it % NSTAGE, b = kb % TC_ABUF;
                    TC_STAMP(1, kb, 2);
                    if constexpr (PAIR) ok = mbar_wait_cluster(&a_ready[b], (kb / TC_ABUF) & 1, deadline);
                    else ok = mbar_wait(&full[s], (it / NSTAGE) & 1, deadline) && mbar_wait(&a_ready[b], (kb / TC_ABUF) & 1, deadline);
                    if (!ok) { *s_error = 1; break; }
                    TC_STAMP(1, kb, 0);
                    tc_fence_after();
                    const uint32_t xaddr = smem_u32(stages + (size_t)s * stage_bytes + 8 * GB + (size_t)(kb & 1) * T * 128);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t desc = tc_smem_desc(xaddr + (uint32_t)(2 * j) * T * 16, (uint32_t)T * 16u, 128u);
                        const uint32_t a_tmem = tmem_base + TC_A_COL0 + b * 32 + j * 8;
                        if constexpr (PAIR) tc_mma_i8_ts_pair(tmem_base, a_tmem, desc, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                        else tc_mma_i8_ts(tmem_base, a_tmem, desc, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    }
                    // once these MMAs retire the activation stage may be refilled and the
                    // weight buffer in tensor memory rewritten (in both CTAs when paired)
                    const bool stage_done = (kb & 1) || kb == KB - 1;
                    if constexpr (PAIR) { if (stage_done) tc_commit_pair(&empty[s]); tc_commit_pair(&a_free[b]); }
                    else { if (stage_done) tc_commit(&empty[s]); tc_commit(&a_free[b]); }
                    TC_STAMP(1, kb, 1);
                }
                if constexpr (PAIR) tc_commit_pair(acc_done); else tc_commit(acc_done);
            }
        } else {
            // ---------------------------------------------------------------- weight unpack -> TMEM
            // A set takes every other STAGE and unpacks both of its k-blocks in one go: one
            // round of barrier waits, eight shared-memory loads, two tensor-memory stores.
            const int q = warp & 3;                       // TMEM lane quarter == weight group of the tile
            const int set = (warp - 2) >> 2;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            bool ok = true;
            const int nstage_iters = (KB + 1) / 2;
            for (int it = set; it < nstage_iters && ok; it += 2) {
                const int s = it % NSTAGE, kb = 2 * it;
                const int kbs = min(2, KB - kb);
                const int b0 = kb % TC_ABUF, b1 = (kb + 1) % TC_ABUF;
                if (q == 2 && lane == 0) TC_STAMP(2, kb, 2);
                ok = mbar_wait(&full[s], (it / NSTAGE) & 1, deadline);
                if (q == 2 && lane == 0) TC_STAMP(2, kb, 3);
                if (ok && kb >= TC_ABUF) {
                    ok = mbar_wait_cluster(&a_free[b0], ((kb / TC_ABUF) - 1) & 1, deadline);
                    if (ok && kbs == 2) ok = mbar_wait_cluster(&a_free[b1], (((kb + 1) / TC_ABUF) - 1) & 1, deadline);
                }
                ok = __all_sync(0xffffffffu, ok);   // the tensor-memory stores below need the whole warp
                if (!ok) { *s_error = 1; break; }
                if (q == 2 && lane == 0) TC_STAMP(2, kb, 0);
                tc_fence_after();
                const uint4* src = reinterpret_cast<const uint4*>(stages + (size_t)s * stage_bytes + q * 2 * GB) + lane;
                if constexpr (W8) {
                    // int8 codes need no unpacking: a lane's 16-byte pieces are already the words of its TMEM row
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (h < kbs) {
                            uint32_t r[32];
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                const uint4 v = src[(8 * h + c) * 32];
                                r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;   // k = 16c + 4j .. +3
                            }
                            tc_st32(lane_addr + TC_A_COL0 + (h ? b1 : b0) * 32, r);
                        }
                    }
                } else {
                uint4 w[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) w[c] = (c < 4 * kbs) ? src[c * 32] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h < kbs) {
                        uint32_t r[32];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t ww[4] = {w[4 * h + c].x, w[4 * h + c].y, w[4 * h + c].z, w[4 * h + c].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                r[c * 8 + j] = (ww[j] << 4) & 0xF0F0F0F0u;       // k = 32c + 4j .. +3      (x16)
                                r[c * 8 + 4 + j] = ww[j] & 0xF0F0F0F0u;          // k = 32c + 16 + 4j .. +3 (x16)
                            }
                        }
                        tc_st32(lane_addr + TC_A_COL0 + (h ? b1 : b0) * 32, r);
                    }
                }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);    // the packed weights of this stage are in registers
                if (q == 2 && lane == 0) TC_STAMP(2, kb, 1);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR && rank != 0) { mbar_arrive_remote(&a_ready[b0], 0); if (kbs == 2) mbar_arrive_remote(&a_ready[b1], 0); }
                    else { mbar_arrive(&a_ready[b0]); if (kbs == 2) mbar_arrive(&a_ready[b1]); }
                }
            }
        }

        // -------------------------------------------------------------------- epilogue
        if (warp >= 2) {
            const int q = warp & 3;
            const int set = (warp - 2) >> 2;              // the two sets take alternate 32-token chunks
            for (int i = tid - 64; i < TOK; i += 32 * TC_UNPACK_WARPS) {
                const int m = tok_base + i;
                s_sx[i] = m < p.M ? p.sx[m] : 0.f;
            }
            if (!mbar_wait_cluster(acc_done, 0, deadline)) *s_error = 1;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const bool done = *reinterpret_cast<volatile int*>(s_error) == 0;   // same answer in all 128 threads
            if (trace && tid == 64) trace[768] = (unsigned long long)(clock64() - c0);
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            // All stages are drained by now: each set of four warps stages its 32-token chunks in
            // 20 KB of the ring so that global stores are 16-byte pieces along the channel axis.
            uint8_t* const stg = stages + (size_t)set * 20480;
            const int ch = q * 32 + lane;
            const int sid = ch;                           // thread index inside the set (0..127)
            int n;                                        // global output channel of this thread
            if (swiglu) n = ch < 64 ? tile * 64 + ch : p.F + tile * 64 + (ch - 64);
            else n = tile * TILE_N + ch;
            const bool n_ok = swiglu ? (tile * 64 + (ch & 63)) < p.F : n < p.N;
            const float sw = n_ok ? p.sw[n] : 0.f;
            const int esize = p.epi == EPI_F16 ? 2 : 4;                       // bytes per output element
            const int row_elems = swiglu ? 64 : 128;                           // outputs per token in this CTA
            const int row_bytes = row_elems * esize + 16;                      // padded staging row
            const int out_cols = swiglu ? p.F : p.N;
            const int col0 = swiglu ? tile * 64 : tile * TILE_N;
            // 16-byte stores need every row start and the tile's first column aligned
            const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.out) & 15u) == 0) && ((size_t)out_cols * esize) % 16 == 0 &&
                                ((size_t)col0 * esize) % 16 == 0;
            for (int t0 = set * 32; t0 < TOK && done; t0 += 64) {
                uint32_t r[32];
                tc_ld32(lane_addr + t0, r);
                tc_wait_ld();
                if (!swiglu) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int v = W8 ? (int)r[i] : (int)r[i] >> 4;   // int4 path: exact, sums are multiples of 16
                        uint8_t* cell = stg + (size_t)i * row_bytes + (size_t)ch * esize;
                        if (p.epi == EPI_I32) *reinterpret_cast<int*>(cell) = v;
                        else {
                            const float y = dequant(v, s_sx[min(t0 + i, TOK - 1)], sw);
                            if (p.epi == EPI_F32) *reinterpret_cast<float*>(cell) = y;
                            else *reinterpret_cast<__half*>(cell) = __float2half_rn(y);
                        }
                    }
                } else {
                    // lanes 64..127 of the accumulator hold the up projection of the same 64
                    // features: hand it to the gate threads through shared memory
                    float* const exch = reinterpret_cast<float*>(stg + 10240);
                    if (ch >= 64) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            exch[i * 64 + (ch - 64)] = dequant(W8 ? (int)r[i] : (int)r[i] >> 4, s_sx[min(t0 + i, TOK - 1)], sw);
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + set) : "memory");
                    if (ch < 64) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int m = tok_base + t0 + i;
                            const float g = dequant(W8 ? (int)r[i] : (int)r[i] >> 4, s_sx[min(t0 + i, TOK - 1)], sw);
                            const float y = __fmul_rn(silu_poly(g), exch[i * 64 + ch]);
                            *reinterpret_cast<float*>(stg + (size_t)i * row_bytes + (size_t)ch * 4) = y;
                            if (p.rowmax) {
                                const bool ok = t0 + i < TOK && m < p.M && n_ok;
                                const uint32_t mx = __reduce_max_sync(0xffffffffu, ok ? (__float_as_uint(y) & 0x7fffffffu) : 0u);
                                if (lane == 0 && mx) atomicMax(&p.rowmax[m], mx);
                            }
                        }
                    }
                }
                asm volatile("bar.sync %0, 128;" ::"r"(2 + set) : "memory");
                // staged chunk -> global: 32 token rows of row_elems outputs
                const int valid_cols = min(row_elems, out_cols - col0);        // > 0 for every launched tile
                if (vec_ok) {
                    const int pieces_per_row = row_elems * esize / 16;
                    for (int pc = sid; pc < 32 * pieces_per_row; pc += 128) {
                        const int i = pc / pieces_per_row, c16 = pc - i * pieces_per_row;
                        const int m = tok_base + t0 + i;
                        const int first = c16 * (16 / esize);
                        if (t0 + i < TOK && m < p.M && first < valid_cols) {
                            const uint4 val = *reinterpret_cast<const uint4*>(stg + (size_t)i * row_bytes + (size_t)c16 * 16);
                            uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + ((size_t)m * out_cols + col0) * esize + (size_t)c16 * 16;
                            if (first + 16 / esize <= valid_cols) *reinterpret_cast<uint4*>(dst) = val;
                            else {
                                const uint8_t* src = stg + (size_t)i * row_bytes + (size_t)c16 * 16;
                                for (int e = 0; e < (valid_cols - first) * esize; ++e) dst[e] = src[e];
                            }
                        }
                    }
                } else {
                    for (int el = sid; el < 32 * row_elems; el += 128) {
                        const int i = el / row_elems, c = el - i * row_elems;
                        const int m = tok_base + t0 + i;
                        if (t0 + i < TOK && m < p.M && c < valid_cols) {
                            const uint8_t* src = stg + (size_t)i * row_bytes + (size_t)c * esize;
                            uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + ((size_t)m * out_cols + col0 + c) * esize;
                            if (esize == 2) *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<const uint16_t*>(src);
                            else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
                        }
                    }
                }
                asm volatile("bar.sync %0, 128;" ::"r"(2 + set) : "memory");
            }
        }
    }

    // ------------------------------------------------------------------------ teardown
    if (trace && tid == 64) trace[769] = (unsigned long long)(clock64() - c0);
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) { cluster_arrive(); cluster_wait(); }   // neither CTA frees tensor memory or leaves while the other may still use it
    if (tid == 0 && *s_error) atomicExch(&p.status->device_error, 1);
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

bool gemm_tc_supported(const GemmParams& p)
{
    // 16 x |sum| must fit int32 (see the packed-weight layout), and the kernel keeps all of K in one CTA.
    return p.M >= 1 && (long long)p.KB * KBLOCK <= 131072;
}

template <bool PAIR, bool W8>
static cudaError_t launch_tc_inst(const GemmParams& p, cudaStream_t stream, bool pdl)
{
    auto kernel = gemm_tc_kernel<PAIR, W8>;
    const size_t widest = 227 * 1024;   // the opt-in limit; each launch asks for what its form needs
    static PerDeviceOnce configured;
    int configured_device = -1;
    if (configured.needed(configured_device)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)widest);
        if (e != cudaSuccess) return e;
        configured.mark(configured_device);
    }
    const int tiles = p.epi == EPI_SWIGLU ? (p.F + 63) / 64 : (p.N + TILE_N - 1) / TILE_N;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(TC_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (PAIR) {
        // CTA pairs along x: two neighbouring channel tiles share one 256-token tile
        cfg.gridDim = dim3((unsigned)((tiles + 1) / 2 * 2), (unsigned)((p.M + 255) / 256), 1);
        cfg.dynamicSmemBytes = tc_smem_bytes(128, tc_stage_count(128, true, W8), 256, W8);
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 2;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    } else {
        cfg.gridDim = dim3((unsigned)tiles, (unsigned)((p.M + p.T - 1) / p.T), 1);
        cfg.dynamicSmemBytes = tc_smem_bytes(p.T, tc_stage_count(p.T, false, W8), p.T, W8);
    }
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

cudaError_t launch_gemm_tc(const GemmParams& p, cudaStream_t stream, bool pdl)
{
    if (p.T < 16 || p.T > 256 || p.T % 16 || !gemm_tc_supported(p)) return cudaErrorInvalidValue;
    const bool pair = p.pair != 0;
    if (pair && p.T != 128) return cudaErrorInvalidValue;
    if (p.w8) return pair ? launch_tc_inst<true, true>(p, stream, pdl) : launch_tc_inst<false, true>(p, stream, pdl);
    return pair ? launch_tc_inst<true, false>(p, stream, pdl) : launch_tc_inst<false, false>(p, stream, pdl);
}

} // namespace rkb200
