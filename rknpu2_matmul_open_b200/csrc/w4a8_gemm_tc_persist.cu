// w4a8_gemm_tc_persist.cu -- persistent two-CTA tcgen05 W4A8 GEMM for large batches (sm_100a).
//
// Same data path as w4a8_gemm_tc.cu (packed int4 weights -> tensor memory as the A operand,
// int8 activation codes as shared-memory B operand, kind::i8 MMA over a CTA pair with
// cta_group::2, int32 accumulators in tensor memory), organised so that nothing but the
// tensor pipe sits on the critical path:
//   * one cluster of two CTAs per SM pair stays resident and walks a list of 256-channel x
//     256-token tiles; barriers, tensor memory and descriptors are set up once;
//   * weights and activations travel through SEPARATE rings of bulk copies.  A weight slot is
//     free again as soon as the unpack warps have read it (the unpacked copy lives in tensor
//     memory), an activation slot when the MMAs that read it retire.  Together the rings hold
//     ten k-blocks of activations and eight of weights per CTA -- all of shared memory -- because
//     the copies (L2 hits) take several MMA-stage times to arrive and the pipe starves on a
//     shallower ring;
//   * eight dedicated epilogue warps read the accumulator out of tensor memory, hand it back
//     after the last read and store straight from registers: the 32 lanes of a warp hold 32
//     neighbouring channels of one token, i.e. 64..128 contiguous bytes per store.  For the
//     SwiGLU epilogue, where finishing a chunk costs far more than reading it, three of the four
//     chunks are parked in an L2-resident scratch so that the tensor pipe gets the accumulator
//     back after four reads;
//   * for SwiGLU the unpack warps place gate channels in lanes 0-15 and the matching up
//     channels in lanes 16-31 of every tensor-memory lane quarter, so the epilogue pairs them
//     with one warp shuffle.
// Outputs: binary16 / fp32 / int32 [M,N], or the fused SwiGLU middle [M,F] fp32 (row maxima
// collected).
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"
#include "w4a8_tc.cuh"

namespace rkb200 {

// activation ring: stages of 2 k-blocks (2 x 16 KB); five deep for int4 weights, three where int8 weights (the
// W8A8 operators) take twice the room in the weight ring
__host__ __device__ constexpr int ps_xa(bool w8) { return w8 ? 3 : 5; }
constexpr int PS_XW = 4;                     // weight ring: stages of 2 k-blocks (4 groups x 2 x 2 KB, or x 4 KB for int8 weights)
constexpr int PS_ABUF = 4;                   // weight buffers in tensor memory, one stage (2 k-blocks, 64 columns) each
constexpr int PS_UNPACK_WARPS = 8;
constexpr int PS_EPI_WARPS = 8;              // two per tensor-memory lane quarter, alternating 32-token chunks
constexpr int PS_UNPACK_WARP0 = 3;           // warp 0: activation producer, 1: MMA issuer, 2: weight producer
constexpr int PS_EPI_WARP0 = PS_UNPACK_WARP0 + PS_UNPACK_WARPS;
constexpr int PS_THREADS = 32 * (PS_EPI_WARP0 + PS_EPI_WARPS);   // 608
constexpr int PS_T = 128;                    // tokens of one CTA's activation tile
constexpr int PS_TOK = 256;                  // tokens of the MMA tile (accumulator columns)
constexpr int PS_A_COL0 = 256;
constexpr int PS_TMEM_COLS = 512;
constexpr size_t PS_XA_BYTES = 2 * (size_t)PS_T * 128;   // 32768
__host__ __device__ constexpr size_t ps_group_bytes(bool w8) { return w8 ? 4096 : 2048; }   // one k-block of one 32-channel group
__host__ __device__ constexpr size_t ps_xw_bytes(bool w8) { return 2 * 4 * ps_group_bytes(w8); }   // 16384 / 32768
__host__ __device__ constexpr int ps_barriers(bool w8) { return 2 * ps_xa(w8) + 2 * PS_XW + 2 * PS_ABUF + 2; }
__host__ __device__ constexpr size_t ps_smem_bytes(bool w8)
{
    return ps_xa(w8) * PS_XA_BYTES + PS_XW * ps_xw_bytes(w8) + 2 * PS_TOK * 4 + ps_barriers(w8) * 8 + 32;
}
constexpr int PS_PARK_INTS = 3 * 32 * 32 * PS_EPI_WARPS;   // per CTA: three parked chunks of 32 sums per epilogue thread (96 KB)
static_assert(ps_smem_bytes(false) <= 232448 && ps_smem_bytes(true) <= 232448, "exceeds the shared memory of one CTA");
static_assert(PS_XW == PS_ABUF, "a weight stage and its tensor-memory buffer share one index");

// W8: the weights are int8 codes in the W8 layout (w8a8_kernels.cu): "unpacking" is a copy into tensor memory and the sums
// are not scaled by 16.
template <bool W8>
__global__ void __launch_bounds__(PS_THREADS, 1) gemm_tc_persist_kernel(const GemmParams p, int num_clusters)
{
    constexpr int PS_XA = ps_xa(W8);
    constexpr size_t PS_XW_BYTES = ps_xw_bytes(W8);
    constexpr uint32_t GB = (uint32_t)ps_group_bytes(W8);
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* const acts = smem;
    uint8_t* const wts = acts + PS_XA * PS_XA_BYTES;
    float* const s_sx = reinterpret_cast<float*>(wts + PS_XW * PS_XW_BYTES);   // token scales of the tile being finished
    uint32_t* const s_tilemax = reinterpret_cast<uint32_t*>(s_sx + PS_TOK);      // SwiGLU: the CTA's row maxima of that tile
    uint64_t* const xfull = reinterpret_cast<uint64_t*>(s_tilemax + PS_TOK);
    uint64_t* const xempty = xfull + PS_XA;
    uint64_t* const wfull = xempty + PS_XA;
    uint64_t* const wempty = wfull + PS_XW;
    uint64_t* const a_ready = wempty + PS_XW;
    uint64_t* const a_free = a_ready + PS_ABUF;
    uint64_t* const acc_full = a_free + PS_ABUF;
    uint64_t* const acc_empty = acc_full + 1;
    uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(acc_empty + 1);
    int* const s_error = reinterpret_cast<int*>(s_tmem + 1);

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();
    const int cluster_id = blockIdx.x >> 1;
    const bool swiglu = p.epi == EPI_SWIGLU;
    const int KB = p.KB, KC = KB * 4;
    const int nst = (KB + 1) / 2;                                      // stage iterations per tile
    const int tiles_n = swiglu ? (p.F + 63) / 64 : (p.N + TILE_N - 1) / TILE_N;
    const int pairs_n = (tiles_n + 1) / 2;
    const int pairs_m = (p.M + PS_TOK - 1) / PS_TOK;
    const int total = pairs_n * pairs_m;
    const unsigned long long deadline = global_ns() + p.timeout_ns;
    // optional cycle stamps of cluster 0's leader: [tile j < 16][8] = MMA wait-begin, MMA first issue,
    // MMA last commit, epilogue acc_full seen, tensor memory handed back, stored, [6] cycles the MMA
    // issuer waited for operands; [128 + 2j] / [129 + 2j] cycles unpack warp 0 waited for weights /
    // for a free tensor-memory buffer, [160 + j] for activations; [200] = clusters in the grid
    unsigned long long* const trace = (p.trace && blockIdx.x == 0) ? p.trace : nullptr;
    const long long c0 = clock64();
#define PS_STAMP(j, slot) do { if (trace && (j) < 16) trace[(j) * 8 + (slot)] = (unsigned long long)(clock64() - c0); } while (0)
    if (trace && tid == 0) trace[200] = (unsigned long long)num_clusters;

    if (tid == 0) {
        for (int s = 0; s < PS_XA; ++s) { mbar_init(&xfull[s], 1); mbar_init(&xempty[s], 1); }
        for (int s = 0; s < PS_XW; ++s) { mbar_init(&wfull[s], 1); mbar_init(&wempty[s], 4); }
        for (int b = 0; b < PS_ABUF; ++b) { mbar_init(&a_ready[b], 8); mbar_init(&a_free[b], 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 2 * PS_EPI_WARPS);   // every epilogue warp of both CTAs
        mbar_fence_init();
        *s_error = 0;
    }
    if (tid < PS_TOK) s_tilemax[tid] = 0u;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(PS_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();   // the peer's barriers and tensor memory exist from here on
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    // ---------------------------------------------------------------- weight producer (warp 2)
    // Weights never change, so the ring is filled before the dependency wait below; the
    // producer's position (tile, stage iteration, count) carries over to the loop after it.
    int wp_t = cluster_id, wp_it = 0, wp_gi = 0;
    auto produce_weights = [&](int limit) -> bool {
        const int w = lane & 3;
        bool ok = true;
        while (wp_t < total && wp_gi < limit) {
            const int tile = 2 * (wp_t % pairs_n) + (int)rank;
            const int group = swiglu ? (w < 2 ? tile * 2 + w : p.F / GROUP + tile * 2 + (w - 2)) : tile * 4 + w;
            const uint8_t* wsrc = p.Wp + (size_t)group * KB * GB;
            const int s = wp_gi % PS_XW;
            const int kbs = min(2, KB - 2 * wp_it);
            if (lane == 0) {
                if (wp_gi >= PS_XW) ok = mbar_wait(&wempty[s], ((wp_gi / PS_XW) - 1) & 1, deadline);
                if (ok) mbar_arrive_expect_tx(&wfull[s], (uint32_t)kbs * 4u * GB);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { *s_error = 1; return false; }
            if (lane < 4) bulk_g2s(wts + (size_t)s * PS_XW_BYTES + w * 2 * GB, wsrc + (size_t)wp_it * 2 * GB, (uint32_t)kbs * GB, &wfull[s]);
            ++wp_gi;
            if (++wp_it == nst) { wp_it = 0; wp_t += num_clusters; }
        }
        return true;
    };
    if (warp == 2) produce_weights(PS_XW);   // the first ring-full needs no free slot
    pdl_wait();       // activation codes, scales and the status word come from the kernel in front
    const bool skip = *reinterpret_cast<volatile const int*>(&p.status->bad_input) != 0;

    if (warp == 2) {
        if (!skip) produce_weights(0x7fffffff);
        else if (lane == 0)   // nobody will consume: let the copies already requested land before leaving
            for (int s = 0; s < wp_gi; ++s)
                if (!mbar_wait(&wfull[s], 0, deadline)) { *s_error = 1; break; }
    } else if (warp == 0) {
        // ---------------------------------------------------------------- activation producer
        bool ok = !skip;
        int gi = 0;
        if (lane == 0) {
            for (int t = cluster_id; t < total && ok; t += num_clusters) {
                const int mt = 2 * (t / pairs_n) + (int)rank;
                const uint8_t* xtile = p.Xq + (size_t)mt * ((size_t)KB * 8) * PS_T * 16;
                for (int it = 0; it < nst && ok; ++it, ++gi) {
                    const int s = gi % PS_XA;
                    const int kbs = min(2, KB - 2 * it);
                    if (gi >= PS_XA) ok = mbar_wait_cluster(&xempty[s], ((gi / PS_XA) - 1) & 1, deadline);
                    if (!ok) { *s_error = 1; break; }
                    mbar_arrive_expect_tx(&xfull[s], (uint32_t)kbs * PS_T * 128u);
                    bulk_g2s(acts + (size_t)s * PS_XA_BYTES, xtile + (size_t)it * PS_XA_BYTES, (uint32_t)kbs * PS_T * 128u, &xfull[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader CTA)
        if (lane == 0 && rank == 0 && !skip) {
            const uint32_t idesc = tc_idesc_s8(256, PS_TOK);
            bool ok = true;
            int gi = 0, j = 0;
            for (int t = cluster_id; t < total && ok; t += num_clusters, ++j) {
                PS_STAMP(j, 0);
                if (j > 0) {   // the epilogue warps of both CTAs have read the previous tile out of tensor memory
                    ok = mbar_wait_cluster(acc_empty, (j - 1) & 1, deadline);
                    if (!ok) { *s_error = 1; break; }
                    tc_fence_after();
                }
                long long waited = 0;
                for (int it = 0; it < nst && ok; ++it) {
                    const int g = gi + it, s = g % PS_XA, b = g % PS_ABUF;
                    const int kbs = min(2, KB - 2 * it);
                    const long long w0 = trace ? clock64() : 0;
                    ok = mbar_wait_cluster(&a_ready[b], (g / PS_ABUF) & 1, deadline);
                    if (trace) waited += clock64() - w0;
                    if (!ok) { *s_error = 1; break; }
                    if (it == 0) PS_STAMP(j, 1);
                    tc_fence_after();
                    const uint32_t xaddr = smem_u32(acts + (size_t)s * PS_XA_BYTES);
                    const uint32_t a_tmem = tmem_base + PS_A_COL0 + b * 64;
                    // k-step q: k-block q / 4 of the stage, 32 k = two 16-byte chunks per token: the descriptor's
                    // address field advances by 2 * PS_T (16-byte units) per step
                    const uint64_t desc0 = tc_smem_desc(xaddr, PS_T * 16u, 128u);
                    tc_mma_i8_ts_pair(tmem_base, a_tmem, desc0, idesc, it > 0 ? 1u : 0u);
#pragma unroll
                    for (int q = 1; q < 4; ++q) tc_mma_i8_ts_pair_acc(tmem_base, a_tmem + q * 8, desc0 + (uint64_t)(q * 2 * PS_T), idesc);
                    if (kbs == 2) {
#pragma unroll
                        for (int q = 4; q < 8; ++q) tc_mma_i8_ts_pair_acc(tmem_base, a_tmem + q * 8, desc0 + (uint64_t)(q * 2 * PS_T), idesc);
                    }
                    tc_commit_pair(&xempty[s]);   // the activation stage may be refilled once these MMAs retire
                    tc_commit_pair(&a_free[b]);   // and the weight buffer rewritten, in both CTAs
                }
                gi += nst;
                tc_commit_pair(acc_full);
                PS_STAMP(j, 2);
                if (trace && j < 16) trace[j * 8 + 6] = (unsigned long long)waited;
            }
        }
    } else if (warp >= PS_UNPACK_WARP0 && warp < PS_EPI_WARP0) {
        // ---------------------------------------------------------------- weight unpack -> TMEM
        const int q = warp & 3;
        const int set = (warp - PS_UNPACK_WARP0) >> 2;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        // which rows of the staged weight groups feed this thread's tensor-memory lane:
        // plain: group q, row lane.  SwiGLU: lanes 0-15 gate rows, lanes 16-31 the matching
        // up rows (staged groups 0,1 = gate, 2,3 = up of the same 64 features).
        const int src_group = swiglu ? (q >> 1) + (lane >= 16 ? 2 : 0) : q;
        const int src_row = swiglu ? (q & 1) * 16 + (lane & 15) : lane;
        bool ok = !skip;
        int gi0 = 0, tj = 0;
        const bool tr = trace && warp == PS_UNPACK_WARP0 && lane == 0;
        for (int t = cluster_id; t < total && ok; t += num_clusters, ++tj) {
            long long wait_full = 0, wait_free = 0, wait_x = 0;
            for (int it = 0; it < nst && ok; ++it) {
                const int g = gi0 + it;
                if ((g & 1) != set) continue;                      // the two sets take alternate stages
                const int s = g % PS_XW, b = s, sa = g % PS_XA;
                const int kbs = min(2, KB - 2 * it);
                const long long w0 = tr ? clock64() : 0;
                ok = mbar_wait(&wfull[s], (g / PS_XW) & 1, deadline);
                const long long w1 = tr ? clock64() : 0;
                if (ok && g >= PS_ABUF) ok = mbar_wait_cluster(&a_free[b], ((g / PS_ABUF) - 1) & 1, deadline);
                if (tr) { wait_full += w1 - w0; wait_free += clock64() - w1; }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { *s_error = 1; break; }
                tc_fence_after();
                const uint4* src = reinterpret_cast<const uint4*>(wts + (size_t)s * PS_XW_BYTES + src_group * 2 * GB) + src_row;
                if constexpr (W8) {
                    // int8 codes: a lane's sixteen 16-byte pieces of the stage are the words of its tensor-memory row in order
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (h < kbs) {
                            uint32_t r[32];
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                const uint4 v = src[(8 * h + c) * 32];
                                r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
                            }
                            if (h == kbs - 1) {
                                __syncwarp();
                                if (lane == 0) mbar_arrive(&wempty[s]);    // the stage has been read into registers
                            }
                            tc_st32(lane_addr + PS_A_COL0 + b * 64 + h * 32, r);
                        }
                    }
                } else {
                uint4 w[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) w[c] = (c < 4 * kbs) ? src[c * 32] : make_uint4(0u, 0u, 0u, 0u);
                __syncwarp();
                if (lane == 0) mbar_arrive(&wempty[s]);            // the packed copy is in registers
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h < kbs) {
                        uint32_t r[32];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t ww[4] = {w[4 * h + c].x, w[4 * h + c].y, w[4 * h + c].z, w[4 * h + c].w};
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) {
                                r[c * 8 + jj] = (ww[jj] << 4) & 0xF0F0F0F0u;
                                r[c * 8 + 4 + jj] = ww[jj] & 0xF0F0F0F0u;
                            }
                        }
                        tc_st32(lane_addr + PS_A_COL0 + b * 64 + h * 32, r);
                    }
                }
                }
                tc_wait_st();
                tc_fence_before();
                // the MMA also reads this stage's activations from both CTAs: vouch for this CTA's copy
                const long long w2 = tr ? clock64() : 0;
                ok = mbar_wait(&xfull[sa], (g / PS_XA) & 1, deadline);
                if (tr) wait_x += clock64() - w2;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { *s_error = 1; break; }
                if (lane == 0) { if (rank != 0) mbar_arrive_remote(&a_ready[b], 0); else mbar_arrive(&a_ready[b]); }
            }
            gi0 += nst;
            if (tr && tj < 16) {
                trace[128 + tj * 2] = (unsigned long long)wait_full;
                trace[128 + tj * 2 + 1] = (unsigned long long)wait_free;
                trace[160 + tj] = (unsigned long long)wait_x;
            }
        }
    } else if (warp >= PS_EPI_WARP0) {
        // ---------------------------------------------------------------- epilogue warps
        const int q = warp & 3;                        // TMEM lane quarter this warp may read
        const int eset = (warp - PS_EPI_WARP0) >> 2;   // takes 32-token chunks eset, eset + 2, ...
        const int sid = (warp - PS_EPI_WARP0) * 32 + lane;   // 0..255 among the epilogue threads
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const int out_cols = swiglu ? p.F : p.N;
        // output column (inside the CTA's tile) this thread's accumulator row belongs to
        const int col = swiglu ? (q >> 1) * 32 + (q & 1) * 16 + (lane & 15) : q * 32 + lane;
        const bool up_lane = swiglu && lane >= 16;
        const int odd = lane & 1;
        const bool quad_ok = (out_cols % 4 == 0) && (reinterpret_cast<uintptr_t>(p.out) & 7u) == 0;
        constexpr int SHIFT = W8 ? 0 : 4;             // int4 records enter the MMA times 16
        const bool small_sums = (long long)KB * KBLOCK * (W8 ? 127 : 7) * 127 < (1ll << 22);
        bool ok = !skip;
        int j = 0;
        for (int t = cluster_id; t < total && ok; t += num_clusters, ++j) {
            const int tile = 2 * (t % pairs_n) + (int)rank;
            const int tok_base = (t / pairs_n) * PS_TOK;
            const int col0 = swiglu ? tile * 64 : tile * TILE_N;
            const int n = col0 + col;
            const bool n_ok = n < out_cols;
            const float sw = n_ok ? p.sw[(up_lane ? p.F : 0) + n] : 0.f;
            float* const sx = s_sx;
            {
                const int m = tok_base + sid;
                sx[sid] = m < p.M ? p.sx[m] : 0.f;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");   // scales staged (the barrier at the end of a tile keeps stragglers out)
            ok = mbar_wait_cluster(acc_full, j & 1, deadline);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { *s_error = 1; break; }
            if (sid == 0) PS_STAMP(j, 3);
            tc_fence_after();
            // The tensor pipe stands still until the accumulator is handed back.  Where finishing a chunk is expensive
            // (`park`: the SwiGLU epilogue, fp32 / int32 stores) the first three chunks are only moved: tensor memory ->
            // registers -> this thread's own slots of a scratch in global memory (it stays in L2); the fourth stays in
            // registers, the accumulator goes back, and then the four chunks are finished, the parked ones read back
            // by the thread that wrote them.
            const bool park = p.partials != nullptr && t + num_clusters < total;   // (nothing waits behind a cluster's last tile)
            int* const park_at = park ? p.partials + (size_t)blockIdx.x * PS_PARK_INTS + sid : nullptr;
            if (park) {
#pragma unroll 1
                for (int c = 0; c < 3; ++c) {
                    const int t0 = eset * 32 + 64 * c;
                    if (tok_base + t0 >= p.M) continue;
                    uint32_t r[32];
                    tc_ld32(lane_addr + t0, r);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) __stcg(park_at + (c * 32 + i) * 256, (int)r[i]);
                }
            }
            long long phase_t = (trace && sid == 0) ? clock64() : 0;
            // (diagnostics) cycles the first epilogue thread spends per phase of finishing, summed over the launch:
            // [176] getting a chunk into registers, [177] scales and conversion, [178] the epilogue proper and its stores
            // (SwiGLU: [180] dequantisation, [181] pairing and SiLU, [182] stores, and [178] what is left: the row maxima)
            auto phase = [&](int which) {
                if (trace && sid == 0) { const long long now = clock64(); trace[176 + which] += (unsigned long long)(now - phase_t); phase_t = now; }
            };
#pragma unroll 1
            for (int k = 0; k < 4; ++k) {
                const int c = park ? (k + 3) & 3 : k;
                const int t0 = eset * 32 + 64 * c;
                const bool live_chunk = tok_base + t0 < p.M;
                uint32_t r[32];
                if (live_chunk) {
                    if (!park || k == 0) {
                        tc_ld32(lane_addr + t0, r);
                        tc_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = (uint32_t)__ldcg(park_at + (c * 32 + i) * 256);
                    }
                }
                if (k == (park ? 0 : 3)) {
                    // ---- this warp is done with tensor memory: the next tile's MMAs may overwrite it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { if (rank != 0) mbar_arrive_remote_relaxed(acc_empty, 0); else mbar_arrive_relaxed(acc_empty); }
                    if (sid == 0) PS_STAMP(j, 4);
                }
                if (!live_chunk) continue;
                phase(0);
                // All loads of a chunk come first, then the arithmetic, then the stores: the compiler
                // may not move a load across a store it cannot prove unrelated, and one store per
                // loop iteration would serialise the whole chunk on the latency of each iteration.
                const int m0 = tok_base + t0;
                float sxr[32];
                {
                    const float4* sx4 = reinterpret_cast<const float4*>(sx + t0);
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 f = sx4[v];
                        sxr[4 * v] = f.x; sxr[4 * v + 1] = f.y; sxr[4 * v + 2] = f.z; sxr[4 * v + 3] = f.w;
                    }
                }
                // int32 sum (a multiple of 16) -> float, rounded to nearest like the conversion instruction.
                // The conversion unit is an eighth as wide as the FP32 pipe and would bound the whole
                // drain, so when the bound K * 7 * 127 keeps every sum below 2^22 the exact
                // magic-number form is used: bits(1.5 * 2^23) + v read as a float is 1.5 * 2^23 + v.
                if (p.epi != EPI_I32) {
                    if (small_sums) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__fsub_rn(__uint_as_float(0x4B400000u + (uint32_t)((int)r[i] >> SHIFT)), 12582912.f));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__int2float_rn((int)r[i] >> SHIFT));
                    }
                }
                phase(1);
                if (p.epi == EPI_F16) {
                    // a lane holds one channel of 32 tokens; neighbouring lanes swap halves so that
                    // every lane stores two neighbouring channels of one token as one 32-bit word
                    __half* const out = reinterpret_cast<__half*>(p.out);
                    uint32_t word[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float y0 = __fmul_rn(__fmul_rn(__uint_as_float(r[2 * i]), sxr[2 * i]), sw);
                        const float y1 = __fmul_rn(__fmul_rn(__uint_as_float(r[2 * i + 1]), sxr[2 * i + 1]), sw);
                        const __half2 h = __floats2half2_rn(y0, y1);
                        word[i] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    // two exchange rounds turn (one channel, 32 tokens) per lane into (four neighbouring
                    // channels, 8 tokens) per lane: lanes 4g..4g+3 end up with tokens 4i + (lane & 3)
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t other = __shfl_xor_sync(0xffffffffu, word[i], 1);
                        word[i] = odd ? __byte_perm(other, word[i], 0x7632) : __byte_perm(word[i], other, 0x5410);
                    }
                    const bool upper = (lane & 2) != 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, upper ? word[2 * i] : word[2 * i + 1], 2);
                        if (upper) word[2 * i] = recv; else word[2 * i + 1] = recv;
                        // now (word[2i], word[2i+1]) = channels n4 .. n4+3 of token m0 + 4i + (lane & 3)
                    }
                    const int n4 = n - (lane & 3);
                    const int mrow = m0 + 2 * (int)upper + odd;
                    __half* const row0 = out + (size_t)mrow * out_cols + n4;
                    if (quad_ok && n4 + 3 < out_cols) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (mrow + 4 * i < p.M) *reinterpret_cast<uint2*>(row0 + (size_t)(4 * i) * out_cols) = make_uint2(word[2 * i], word[2 * i + 1]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (mrow + 4 * i < p.M) {
                                __half* dst = row0 + (size_t)(4 * i) * out_cols;
                                const uint32_t ww[2] = {word[2 * i], word[2 * i + 1]};
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    if (n4 + e < out_cols) dst[e] = __ushort_as_half((unsigned short)((ww[e >> 1] >> (16 * (e & 1))) & 0xffffu));
                            }
                    }
                } else if (p.epi == EPI_F32 || p.epi == EPI_I32) {
                    const bool f32 = p.epi == EPI_F32;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        r[i] = f32 ? __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r[i]), sxr[i]), sw)) : (uint32_t)((int)r[i] >> SHIFT);
                    }
                    uint32_t* const row0 = reinterpret_cast<uint32_t*>(p.out) + (size_t)m0 * out_cols + n;
                    if (n_ok) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (m0 + i < p.M) row0[(size_t)i * out_cols] = r[i];
                    }
                } else {
                    // Lanes 0-15 hold the gate rows g, lanes 16-31 the matching up rows u of 16 features.  For
                    // every token pair the halves swap what the other needs, so that the gate lanes finish the
                    // even token and the up lanes the odd one: each lane evaluates 16 SiLUs instead of 32.
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r[i]), sxr[i]), sw));
                    float y[16];
                    uint32_t mx[16];
                    const int mine_row = m0 + (up_lane ? 1 : 0);
                    phase(4);
#pragma unroll
                    for (int i0 = 0; i0 < 16; i0 += 4) {     // four tokens in lock step (see silu_poly4)
                        float g4[4], u4[4], s4[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int i = i0 + k;
                            const float a0 = __uint_as_float(r[2 * i]), a1 = __uint_as_float(r[2 * i + 1]);
                            const float o0 = __shfl_xor_sync(0xffffffffu, a0, 16);   // gate lanes: u of token 2i; up lanes: g of token 2i
                            const float o1 = __shfl_xor_sync(0xffffffffu, a1, 16);   // gate lanes: u of token 2i+1; up lanes: g of token 2i+1
                            g4[k] = up_lane ? o1 : a0;
                            u4[k] = up_lane ? a1 : o0;
                        }
                        silu_poly4(g4, s4);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int i = i0 + k;
                            y[i] = __fmul_rn(s4[k], u4[k]);
                            const bool live = n_ok && mine_row + 2 * i < p.M;
                            mx[i] = live ? (__float_as_uint(y[i]) & 0x7fffffffu) : 0u;
                        }
                    }
                    phase(5);
                    float* const row0 = reinterpret_cast<float*>(p.out) + (size_t)mine_row * out_cols + n;
                    if (n_ok) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (mine_row + 2 * i < p.M) row0[(size_t)(2 * i) * out_cols] = y[i];
                    }
                    phase(6);
                    if (p.rowmax) {
                        // Maxima over the 16 lanes of each half, one token per value: a folding exchange that halves
                        // the values a lane holds at every step (8 + 4 + 2 + 1 shuffles instead of 16 x 4); lane l of
                        // a half ends up with the maximum of token l & 15 and issues that token's one atomic.
#pragma unroll
                        for (int width = 8; width > 0; width >>= 1) {
                            const bool upper = (lane & width) != 0;
#pragma unroll
                            for (int k = 0; k < width; ++k) {
                                const uint32_t keep = upper ? mx[k + width] : mx[k];
                                const uint32_t give = upper ? mx[k] : mx[k + width];
                                mx[k] = max(keep, __shfl_xor_sync(0xffffffffu, give, width));
                            }
                        }
                        // collected per CTA and tile in shared memory first: one global atomic per token and tile
                        // instead of one per token, tile and 16 features
                        if (mx[0]) atomicMax(&s_tilemax[t0 + (up_lane ? 1 : 0) + 2 * (lane & 15)], mx[0]);
                    }
                }
                phase(2);
            }
            if (sid == 0) PS_STAMP(j, 5);
            asm volatile("bar.sync 1, 256;" ::: "memory");   // every epilogue warp is done with this tile's scales and maxima
            phase(3);
            if (swiglu && p.rowmax) {
                const uint32_t m = s_tilemax[sid];
                if (m) {
                    atomicMax(&p.rowmax[tok_base + sid], m);
                    s_tilemax[sid] = 0u;
                }
            }
        }
    }

    // ------------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();   // neither CTA frees tensor memory or leaves while the other may still use it
    if (tid == 0 && *s_error) atomicExch(&p.status->device_error, 1);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(PS_TMEM_COLS) : "memory");
    }
}

bool gemm_tc_persist_supported(const GemmParams& p)
{
    return p.pair && p.T == PS_T && (long long)p.KB * KBLOCK <= 131072;
}

size_t gemm_tc_persist_park_bytes(int sm_count) { return size_t(sm_count) * PS_PARK_INTS * sizeof(int); }

template <bool W8>
static cudaError_t launch_persist_inst(const GemmParams& p, cudaStream_t stream, bool pdl)
{
    auto kernel = gemm_tc_persist_kernel<W8>;
    static PerDeviceOnce configured;
    static int clusters_of_device[64] = {};   // resident CTA pairs, per CUDA ordinal
    int device = -1;
    int max_clusters = 0;
    const bool setup = configured.needed(device);
    if (!setup) max_clusters = clusters_of_device[device];
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(PS_THREADS);
    cfg.dynamicSmemBytes = ps_smem_bytes(W8);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    if (setup || !max_clusters) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ps_smem_bytes(W8));
        if (e != cudaSuccess) return e;
        // how many CTA pairs can be resident at once: the grid is exactly that many
        cfg.gridDim = dim3(2, 1, 1);
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
        if (e != cudaSuccess || n < 1) { cudaGetLastError(); int dev = 0, sms = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); n = sms / 2; }
        max_clusters = n;
        if (device >= 0 && device < 64) { clusters_of_device[device] = n; configured.mark(device); }
    }
    const int tiles_n = p.epi == EPI_SWIGLU ? (p.F + 63) / 64 : (p.N + TILE_N - 1) / TILE_N;
    const int total = ((tiles_n + 1) / 2) * ((p.M + PS_TOK - 1) / PS_TOK);
    const int clusters = total < max_clusters ? total : max_clusters;
    cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
    int n = 1;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, p, clusters);
}

cudaError_t launch_gemm_tc_persist(const GemmParams& p, cudaStream_t stream, bool pdl)
{
    if (!gemm_tc_persist_supported(p)) return cudaErrorInvalidValue;
    return p.w8 ? launch_persist_inst<true>(p, stream, pdl) : launch_persist_inst<false>(p, stream, pdl);
}

} // namespace rkb200
