// w4a8_gemm_tc_persist.cu -- persistent two-CTA tcgen05 W4A8 GEMM for large batches (sm_100a).
//
// Same data path as w4a8_gemm_tc.cu (packed int4 weights -> tensor memory as the A operand,
// int8 activation codes as shared-memory B operand, kind::i8 MMA over a CTA pair with
// cta_group::2, int32 accumulators in tensor memory), organised so that nothing but the
// tensor pipe sits on the critical path between tiles:
//   * one cluster of two CTAs per SM pair stays resident and walks a list of 256-channel x
//     256-token tiles; barriers, tensor memory and descriptors are set up once;
//   * eight dedicated epilogue warps drain the accumulator into a staging buffer in shared
//     memory (converted to the output type), hand the tensor memory back, and only then
//     write the staged tile to global memory in 16-byte pieces -- while the producer, the
//     unpack warps and the MMA issuer are already deep in the next tile;
//   * for SwiGLU the unpack warps place gate channels in lanes 0-15 and the matching up
//     channels in lanes 16-31 of every tensor-memory lane quarter, so the epilogue pairs them
//     with one warp shuffle.
// Outputs: binary16 [M,N], or the fused SwiGLU middle [M,F] fp32 (row maxima collected).
// Plain fp32 / int32 outputs (twice the staging size) use the non-persistent kernel.
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"
#include "w4a8_tc.cuh"

namespace rkb200 {

constexpr int PS_STAGES = 3;                 // x 2 k-blocks x (8 KB weights + 16 KB activations)
constexpr int PS_ABUF = 4;                   // weight buffers in tensor memory, one STAGE (2 k-blocks, 64 columns) each
constexpr int PS_UNPACK_WARPS = 8;
constexpr int PS_EPI_WARPS = 8;              // two per tensor-memory lane quarter, alternating 32-token chunks
constexpr int PS_THREADS = 64 + 32 * PS_UNPACK_WARPS + 32 * PS_EPI_WARPS;   // 576
constexpr int PS_T = 128;                    // tokens of one CTA's activation tile
constexpr int PS_TOK = 256;                  // tokens of the MMA tile (accumulator columns)
constexpr int PS_A_COL0 = 256;
constexpr int PS_TMEM_COLS = 512;
constexpr size_t PS_STAGE_BYTES = 2 * (8192 + (size_t)PS_T * 128);          // 49152
// Staging is channel-major so that a draining thread (one channel, 32 tokens per chunk) writes
// 16-byte vectors: 128 rows of 256 x f16 (512 B), or 64 rows of 256 x fp32 (1024 B) for SwiGLU,
// each row padded by 16 B so that the 32 lanes of a warp spread over all banks.
constexpr int PS_ROW_F16 = 512 + 16;
constexpr int PS_ROW_F32 = 1024 + 16;
constexpr size_t PS_STAGING_BYTES = 128 * PS_ROW_F16;   // 67584 >= 64 * PS_ROW_F32
constexpr size_t PS_SMEM_BYTES = PS_STAGES * PS_STAGE_BYTES + PS_STAGING_BYTES + PS_TOK * 4 +
                                 (2 * PS_STAGES + 2 * PS_ABUF + 2) * 8 + 32;

__global__ void __launch_bounds__(PS_THREADS, 1) gemm_tc_persist_kernel(const GemmParams p, int num_clusters)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* const stages = smem;
    uint8_t* const staging = stages + PS_STAGES * PS_STAGE_BYTES;
    float* const s_sx = reinterpret_cast<float*>(staging + PS_STAGING_BYTES);
    uint64_t* const full = reinterpret_cast<uint64_t*>(s_sx + PS_TOK);
    uint64_t* const empty = full + PS_STAGES;
    uint64_t* const a_ready = empty + PS_STAGES;
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
    // MMA last commit, epilogue acc_full seen, drained, stored; [200] = clusters in the grid
    unsigned long long* const trace = (p.trace && blockIdx.x == 0) ? p.trace : nullptr;
    const long long c0 = clock64();
#define PS_STAMP(j, slot) do { if (trace && (j) < 16) trace[(j) * 8 + (slot)] = (unsigned long long)(clock64() - c0); } while (0)
    if (trace && tid == 0) trace[200] = (unsigned long long)num_clusters;

    if (tid == 0) {
        for (int s = 0; s < PS_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 5); }
        for (int b = 0; b < PS_ABUF; ++b) { mbar_init(&a_ready[b], 8); mbar_init(&a_free[b], 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 2 * PS_EPI_WARPS);   // every epilogue warp of both CTAs
        mbar_fence_init();
        *s_error = 0;
    }
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
    pdl_wait();       // activation codes, scales and the status word come from the kernel in front
    const bool skip = *reinterpret_cast<volatile const int*>(&p.status->bad_input) != 0;

    if (!skip) {
        if (warp == 0) {
            // ---------------------------------------------------------------- producer
            const int w = lane & 3;
            bool ok = true;
            int gi = 0;                                                 // stage iterations issued so far
            for (int t = cluster_id; t < total && ok; t += num_clusters) {
                const int tile = 2 * (t % pairs_n) + (int)rank, mt = 2 * (t / pairs_n) + (int)rank;
                const int group = swiglu ? (w < 2 ? tile * 2 + w : p.F / GROUP + tile * 2 + (w - 2)) : tile * 4 + w;
                const uint8_t* wsrc = p.Wp + (size_t)group * KC * 512;
                const uint8_t* xtile = p.Xq + (size_t)mt * ((size_t)KB * 8) * PS_T * 16;
                for (int it = 0; it < nst && ok; ++it, ++gi) {
                    const int s = gi % PS_STAGES;
                    const int kbs = min(2, KB - 2 * it);
                    if (lane == 0) {
                        if (gi >= PS_STAGES) ok = mbar_wait_cluster(&empty[s], ((gi / PS_STAGES) - 1) & 1, deadline);
                        if (ok) mbar_arrive_expect_tx(&full[s], (uint32_t)kbs * (8192u + PS_T * 128u));
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) { *s_error = 1; break; }
                    uint8_t* dst = stages + (size_t)s * PS_STAGE_BYTES;
                    if (lane < 4) bulk_g2s(dst + w * 4096, wsrc + (size_t)it * 4096, (uint32_t)kbs * 2048u, &full[s]);
                    else if (lane == 4) bulk_g2s(dst + 16384, xtile + (size_t)it * 16 * PS_T * 16, (uint32_t)kbs * PS_T * 128u, &full[s]);
                }
            }
        } else if (warp == 1) {
            // ---------------------------------------------------------------- MMA issuer (leader CTA)
            if (lane == 0 && rank == 0) {
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
                        const int g = gi + it, s = g % PS_STAGES, b = g % PS_ABUF;
                        const int kbs = min(2, KB - 2 * it);
                        const long long w0 = trace ? clock64() : 0;
                        ok = mbar_wait_cluster(&a_ready[b], (g / PS_ABUF) & 1, deadline);
                        if (trace) waited += clock64() - w0;
                        if (!ok) { *s_error = 1; break; }
                        if (it == 0) PS_STAMP(j, 1);
                        tc_fence_after();
                        const uint32_t xaddr = smem_u32(stages + (size_t)s * PS_STAGE_BYTES + 16384);
                        const uint32_t a_tmem = tmem_base + PS_A_COL0 + b * 64;
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            if (q < 4 * kbs) {
                                // k-step q: half q/4 of the stage, 32 k = two 16-byte chunks per token
                                const uint64_t desc = tc_smem_desc(xaddr + (uint32_t)(q >> 2) * PS_T * 128 + (uint32_t)(2 * (q & 3)) * PS_T * 16, PS_T * 16u, 128u);
                                tc_mma_i8_ts_pair(tmem_base, a_tmem + q * 8, desc, idesc, (it > 0 || q > 0) ? 1u : 0u);
                            }
                        }
                        tc_commit_pair(&empty[s]);    // the activation stage may be refilled once these MMAs retire
                        tc_commit_pair(&a_free[b]);   // and the weight buffer rewritten, in both CTAs
                    }
                    gi += nst;
                    tc_commit_pair(acc_full);
                    PS_STAMP(j, 2);
                    if (trace && j < 16) trace[j * 8 + 6] = (unsigned long long)waited;   // cycles spent waiting for weights in tensor memory
                }
            }
        } else if (warp < 2 + PS_UNPACK_WARPS) {
            // ---------------------------------------------------------------- weight unpack -> TMEM
            const int q = warp & 3;
            const int set = (warp - 2) >> 2;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            // which rows of the staged weight groups feed this thread's tensor-memory lane:
            // plain: group q, row lane.  SwiGLU: lanes 0-15 gate rows, lanes 16-31 the matching
            // up rows (staged groups 0,1 = gate, 2,3 = up of the same 64 features).
            const int src_group = swiglu ? (q >> 1) + (lane >= 16 ? 2 : 0) : q;
            const int src_row = swiglu ? (q & 1) * 16 + (lane & 15) : lane;
            bool ok = true;
            int gi0 = 0, tj = 0;
            const bool tr = trace && warp == 2 && lane == 0;
            for (int t = cluster_id; t < total && ok; t += num_clusters, ++tj) {
                long long wait_full = 0, wait_free = 0;
                for (int it = 0; it < nst && ok; ++it) {
                    const int g = gi0 + it;
                    if ((g & 1) != set) continue;                      // the two sets take alternate stages
                    const int s = g % PS_STAGES, b = g % PS_ABUF;
                    const int kbs = min(2, KB - 2 * it);
                    const long long w0 = tr ? clock64() : 0;
                    ok = mbar_wait(&full[s], (g / PS_STAGES) & 1, deadline);
                    const long long w1 = tr ? clock64() : 0;
                    if (ok && g >= PS_ABUF) ok = mbar_wait_cluster(&a_free[b], ((g / PS_ABUF) - 1) & 1, deadline);
                    if (tr) { wait_full += w1 - w0; wait_free += clock64() - w1; }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) { *s_error = 1; break; }
                    tc_fence_after();
                    const uint4* src = reinterpret_cast<const uint4*>(stages + (size_t)s * PS_STAGE_BYTES + src_group * 4096) + src_row;
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
                                for (int jj = 0; jj < 4; ++jj) {
                                    r[c * 8 + jj] = (ww[jj] << 4) & 0xF0F0F0F0u;
                                    r[c * 8 + 4 + jj] = ww[jj] & 0xF0F0F0F0u;
                                }
                            }
                            tc_st32(lane_addr + PS_A_COL0 + b * 64 + h * 32, r);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[s]);
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { if (rank != 0) mbar_arrive_remote(&a_ready[b], 0); else mbar_arrive(&a_ready[b]); }
                }
                gi0 += nst;
                if (tr && tj < 16) { trace[128 + tj * 2] = (unsigned long long)wait_full; trace[128 + tj * 2 + 1] = (unsigned long long)wait_free; }
            }
        } else {
            // ---------------------------------------------------------------- epilogue warps
            const int q = warp & 3;                        // TMEM lane quarter this warp may read
            const int eset = (warp - 2 - PS_UNPACK_WARPS) >> 2;          // takes 32-token chunks eset, eset + 2, ...
            const int sid = (warp - 2 - PS_UNPACK_WARPS) * 32 + lane;   // 0..255 among the epilogue threads
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            const int esize = swiglu ? 4 : 2;
            const int row_elems = swiglu ? 64 : 128;       // outputs per token of this CTA
            const int out_cols = swiglu ? p.F : p.N;
            // output column (inside the CTA's tile) this thread's accumulator row belongs to
            const int col = swiglu ? (q >> 1) * 32 + (q & 1) * 16 + (lane & 15) : q * 32 + lane;
            const bool up_lane = swiglu && lane >= 16;
            bool ok = true;
            int j = 0;
            for (int t = cluster_id; t < total && ok; t += num_clusters, ++j) {
                const int tile = 2 * (t % pairs_n) + (int)rank;
                const int tok_base = (t / pairs_n) * PS_TOK;
                const int col0 = swiglu ? tile * 64 : tile * TILE_N;
                const bool n_ok = col0 + col < out_cols;
                const float sw = n_ok ? p.sw[(up_lane ? p.F : 0) + col0 + col] : 0.f;
                for (int i = sid; i < PS_TOK; i += 32 * PS_EPI_WARPS) {
                    const int m = tok_base + i;
                    s_sx[i] = m < p.M ? p.sx[m] : 0.f;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");   // scales staged; previous tile's staging is free
                ok = mbar_wait_cluster(acc_full, j & 1, deadline);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { *s_error = 1; break; }
                if (sid == 0) PS_STAMP(j, 3);
                tc_fence_after();
                // ---- drain tensor memory into the staging buffer (converted, channel-major)
                for (int t0 = eset * 32; t0 < PS_TOK; t0 += 64) {
                    uint32_t r[32];
                    tc_ld32(lane_addr + t0, r);
                    tc_wait_ld();
                    if (!swiglu) {
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float y0 = dequant((int)r[2 * i] >> 4, s_sx[t0 + 2 * i], sw);
                            const float y1 = dequant((int)r[2 * i + 1] >> 4, s_sx[t0 + 2 * i + 1], sw);
                            const __half2 h = __floats2half2_rn(y0, y1);
                            packed[i] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(staging + (size_t)col * PS_ROW_F16 + (size_t)t0 * 2);
#pragma unroll
                        for (int v = 0; v < 4; ++v) dst[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                    } else {
                        float y[32];
                        uint32_t mx[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float mine = dequant((int)r[i] >> 4, s_sx[t0 + i], sw);     // gate lanes: g, up lanes: u
                            const float up = __shfl_xor_sync(0xffffffffu, mine, 16);
                            y[i] = __fmul_rn(silu_poly(mine), up);                              // meaningful in gate lanes
                            const bool live = !up_lane && n_ok && tok_base + t0 + i < p.M;
                            mx[i] = live ? (__float_as_uint(y[i]) & 0x7fffffffu) : 0u;
                        }
                        if (!up_lane) {
                            uint4* dst = reinterpret_cast<uint4*>(staging + (size_t)col * PS_ROW_F32 + (size_t)t0 * 4);
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                dst[v] = make_uint4(__float_as_uint(y[4 * v]), __float_as_uint(y[4 * v + 1]), __float_as_uint(y[4 * v + 2]),
                                                    __float_as_uint(y[4 * v + 3]));
                        }
                        if (p.rowmax) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const uint32_t m32 = __reduce_max_sync(0xffffffffu, mx[i]);
                                if (lane == 0 && m32) atomicMax(&p.rowmax[tok_base + t0 + i], m32);
                            }
                        }
                    }
                }
                // ---- tensor memory is free again: the next tile's MMAs may overwrite it
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { if (rank != 0) mbar_arrive_remote(acc_empty, 0); else mbar_arrive(acc_empty); }
                asm volatile("bar.sync 1, 256;" ::: "memory");   // the whole tile is staged
                if (sid == 0) PS_STAMP(j, 4);
                // ---- staged tile -> global memory: a 16-byte piece = 8 (f16) or 4 (fp32) neighbouring
                // columns of one token, gathered from as many staging rows
                const int valid_cols = min(row_elems, out_cols - col0);
                const int per_piece = 16 / esize;
                const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.out) & 15u) == 0) && ((size_t)out_cols * esize) % 16 == 0 &&
                                    ((size_t)col0 * esize) % 16 == 0;
                if (valid_cols > 0) {
                    for (int pc = sid; pc < PS_TOK * 16; pc += 32 * PS_EPI_WARPS) {
                        const int c16 = pc >> 8, i = pc & 255;          // consecutive threads: consecutive tokens (conflict-free reads)
                        const int m = tok_base + i;
                        const int first = c16 * per_piece;
                        if (m >= p.M || first >= valid_cols) continue;
                        uint32_t wv[4];
                        if (!swiglu) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const uint32_t lo = *reinterpret_cast<const uint16_t*>(staging + (size_t)(first + 2 * e) * PS_ROW_F16 + (size_t)i * 2);
                                const uint32_t hi = *reinterpret_cast<const uint16_t*>(staging + (size_t)(first + 2 * e + 1) * PS_ROW_F16 + (size_t)i * 2);
                                wv[e] = lo | (hi << 16);
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) wv[e] = *reinterpret_cast<const uint32_t*>(staging + (size_t)(first + e) * PS_ROW_F32 + (size_t)i * 4);
                        }
                        uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + ((size_t)m * out_cols + col0 + first) * esize;
                        if (vec_ok && first + per_piece <= valid_cols) *reinterpret_cast<uint4*>(dst) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                        else {
                            const uint8_t* src = reinterpret_cast<const uint8_t*>(wv);
                            const int nbytes = min(per_piece, valid_cols - first) * esize;
                            for (int e = 0; e < nbytes; ++e) dst[e] = src[e];
                        }
                    }
                }
                if (sid == 0) PS_STAMP(j, 5);
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
    return p.pair && p.T == PS_T && (p.epi == EPI_F16 || p.epi == EPI_SWIGLU) && (long long)p.KB * KBLOCK <= 131072;
}

cudaError_t launch_gemm_tc_persist(const GemmParams& p, cudaStream_t stream, bool pdl)
{
    if (!gemm_tc_persist_supported(p)) return cudaErrorInvalidValue;
    static int max_clusters = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(PS_THREADS);
    cfg.dynamicSmemBytes = PS_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    if (!max_clusters) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PS_SMEM_BYTES);
        if (e != cudaSuccess) return e;
        // how many CTA pairs can be resident at once: the grid is exactly that many
        cfg.gridDim = dim3(2, 1, 1);
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_persist_kernel, &cfg);
        if (e != cudaSuccess || n < 1) { cudaGetLastError(); int dev = 0, sms = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); n = sms / 2; }
        max_clusters = n;
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
    return cudaLaunchKernelEx(&cfg, gemm_tc_persist_kernel, p, clusters);
}

} // namespace rkb200
