// w4a8_fused.cu -- single-kernel W4A8 linear for small batches (decode, M <= 32) on sm_100a.
//
// One launch does what the reference does in three stages (scan + quantise, src/
// rk_npu_w4a8_quant.cpp:52-135; contraction; reconstruct + dequantise, src/
// rk_npu_w4a8_output.cpp:35-161), so a dependent chain of small linears pays one kernel
// of latency per linear and the weight stream of the next launch (requested before the
// programmatic dependency wait) overlaps the dependent tail of the current one.
//
// A CTA owns 128 output channels and one K slice; the CTAs of a slice set form a cluster
// along y.  Per CTA:
//   1. thread 0 requests every weight k-block of the slice with bulk async copies
//      (weights are immutable, so this happens before waiting for the producer of A);
//   2. max |A| over the CTA's K slice per token, pushed to every CTA of the cluster through
//      distributed shared memory; one cluster barrier later every CTA holds the full-row
//      maximum and derives the same scale;
//   3. the slice of A is quantised into shared memory in the layout the mma.sync B fragments
//      read; 4. int8 mma.sync over the slice; 5. partial sums are pushed to the cluster rank
//      that owns each channel, one more cluster barrier, local sum, dequantise / SwiGLU, store.
// A launch whose CTAs would fill more shared memory than the launches around it leave free runs
// two column tiles per CTA (tiles_per_cta = 2): half the CTAs, all resident at once beside their
// neighbours; steps 1-3 are shared, the second tile's weights are requested into the first tile's
// place once its contraction has read them, and steps 4-5 of the first tile hide their arrival.
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace rkb200 {

__host__ __device__ constexpr size_t fused_smem_bytes(int tc, int stages, int tiles_per_cta)
{
    return (size_t)stages * 8192                       // weight k-blocks
           + (size_t)stages * tc * 128                 // activation codes of the slice
           + (size_t)tiles_per_cta * tc * 192 * 4      // inbox per tile: partial sums for the channels this rank owns
           + (size_t)8 * tc * 4                        // inbox: per-rank partial row maxima
           + (size_t)4 * tc * 4                        // row max, scale, inverse, SwiGLU row max
           + 128 * 4 + 40 + 16;                        // channel scales, five barriers, flags
}

constexpr size_t FUSED_SMEM_LIMIT = 227 * 1024;   // dynamic shared memory one CTA may ask for
constexpr int FUSED_THREADS = 256;   // eight warps: (weight group, m16 tile) pairs in the contraction

template <int NT, bool HALF>
__global__ void __launch_bounds__(FUSED_THREADS) gemm_fused_kernel(const FusedParams p)
{
    using AT = typename ActType<HALF>::type;
    constexpr int TC = 8 * NT;
    extern __shared__ __align__(128) uint8_t smem[];
    const int nst = p.stages;
    uint8_t* const wst = smem;
    uint8_t* const xs = wst + (size_t)nst * 8192;
    const int TPC = p.tiles_per_cta;                   // 1 or 2 column tiles per CTA, one after the other
    int32_t* const inbox_all = reinterpret_cast<int32_t*>(xs + (size_t)nst * TC * 128);
    uint32_t* const inbox_max = reinterpret_cast<uint32_t*>(inbox_all + TPC * TC * 192);
    uint32_t* const s_max = inbox_max + 8 * TC;
    float* const s_scale = reinterpret_cast<float*>(s_max + TC);
    float* const s_inv = s_scale + TC;
    uint32_t* const s_outmax = reinterpret_cast<uint32_t*>(s_inv + TC);
    float* const s_sw = reinterpret_cast<float*>(s_outmax + TC);   // 128 channel scales of this CTA
    // barriers, each used for one phase only: [0] row maxima of all ranks, [1 + i] weights of tile i landed,
    // [3 + i] partial sums of tile i
    uint64_t* const full = reinterpret_cast<uint64_t*>(s_sw + 128);
    int* const s_flags = reinterpret_cast<int*>(full + 5);   // [0] bad verdict, [1] wait ran out

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rank = blockIdx.y, S = p.split;
    const int tiles_total = p.epi == EPI_SWIGLU ? (p.F + 63) / 64 : (p.N + TILE_N - 1) / TILE_N;
    const int tile_first = blockIdx.x * TPC;
    const int ntile = min(TPC, tiles_total - tile_first);   // the last CTA of an odd count has one tile
    unsigned long long* const trace = (p.trace && tid == 0) ? p.trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 8 : nullptr;
    const long long c_start = clock64();
    if (trace) trace[0] = global_ns();
    const bool swiglu = p.epi == EPI_SWIGLU;
    const int KC = p.KB * 4;
    const int kb0 = (int)(((long long)p.KB * rank) / S), kb1 = (int)(((long long)p.KB * (rank + 1)) / S);
    const int nkb = kb1 - kb0;
    const unsigned long long deadline = global_ns() + p.timeout_ns;
    cg::cluster_group cluster = cg::this_cluster();

    // Weights of the slice: per group one contiguous run of nkb k-blocks -> four bulk
    // copies on one barrier, requested before the dependency wait (weights never change).
    if (tid == 0) {
        for (int b = 0; b < 5; ++b) mbar_init(&full[b], 1);
        mbar_fence_init();
        if (S > 1 && p.rowmax_in == nullptr) mbar_arrive_expect_tx(&full[0], (uint32_t)(S * TC * 4));
        s_flags[0] = 0;
        s_flags[1] = 0;
        if (nkb > 0) mbar_arrive_expect_tx(&full[1], (uint32_t)nkb * 8192u);
    }
    if (tid < TC) { s_max[tid] = 0u; s_outmax[tid] = 0u; }
    if (S > 1) cluster_arrive();   // matched by the wait in front of the first remote store
    __syncthreads();
    // four bulk copies bring one tile's weight slice (per group one contiguous run of nkb k-blocks)
    auto request_weights = [&](int tile, uint64_t* bar) {
        const int w = tid;
        const int group = swiglu ? (w < 2 ? tile * 2 + w : p.F / GROUP + tile * 2 + (w - 2)) : tile * 4 + w;
        bulk_g2s(wst + (size_t)w * nkb * 2048, p.Wp + ((size_t)group * KC + (size_t)kb0 * 4) * 512, (uint32_t)nkb * 2048u, bar);
    };
    // channel scales of a tile's outputs (constants)
    auto stage_channel_scales = [&](int tile) {
        if (tid < 128) {
            const int n0 = swiglu ? (tid < 64 ? tile * 64 + tid : p.F + tile * 64 + (tid - 64)) : tile * TILE_N + tid;
            s_sw[tid] = n0 < p.NG * GROUP ? p.sw[n0] : 0.f;
        }
    };
    if (tid < 4 && nkb > 0) request_weights(tile_first, &full[1]);
    stage_channel_scales(tile_first);
    // ---- 1. row maxima over this CTA's K slice.  Work item = (token, 16-element unit);
    // the first UMAX items of a thread stay in registers for the quantisation pass.  Where they lie is
    // settled before the dependency wait, so that no integer division sits between "A exists" and the loads.
    const int k_begin = kb0 * KBLOCK;
    const int units = nkb * 8;                          // 16-element units per token in the slice
    const AT* A = reinterpret_cast<const AT*>(p.A);
    const bool vec = (reinterpret_cast<uintptr_t>(A) & 15u) == 0 && (p.K % (HALF ? 8 : 4)) == 0;
    constexpr int UMAX = HALF ? 2 : 1;
    Raw16<HALF> kept[UMAX];
    const int items = TC * units;
    const bool warp_one_token = (units & 31) == 0;
    int pos_tok[UMAX], pos_u[UMAX];
#pragma unroll
    for (int it = 0; it < UMAX; ++it) {
        const int idx = tid + FUSED_THREADS * it;
        pos_tok[it] = units > 0 ? idx / units : 0;
        pos_u[it] = idx - pos_tok[it] * units;
    }
    if (trace) trace[1] = (unsigned long long)(clock64() - c_start);
    pdl_wait();   // the producer of A (and of the row maxima) has finished
    if (trace) trace[2] = (unsigned long long)(clock64() - c_start);
#pragma unroll
    for (int it = 0; it < UMAX; ++it) {
        const int idx = tid + FUSED_THREADS * it;
        const int tok = pos_tok[it], u = pos_u[it];
        const int k0 = k_begin + u * 16;
#pragma unroll
        for (int i = 0; i < (HALF ? 8 : 16); ++i) kept[it].w[i] = 0u;
        uint32_t bits = 0;
        if (idx < items && tok < p.M && k0 < p.K) {
            load_raw<HALF>(A + (size_t)tok * p.K, k0, p.K, vec, kept[it]);
            bits = raw_maxbits<HALF>(kept[it]);
        }
        if (p.rowmax_in == nullptr) {
            // 256 threads hammering eight shared words serialise; when a warp's 32 items belong to one
            // token (units a multiple of 32) the warp reduces first and issues one atomic
            if (warp_one_token) {
                bits = __reduce_max_sync(0xffffffffu, bits);
                if (lane == 0 && bits) atomicMax(&s_max[min(tok, TC - 1)], bits);
            } else if (bits) atomicMax(&s_max[tok], bits);
        }
    }
    if (p.rowmax_in == nullptr) {
        for (int idx = tid + FUSED_THREADS * UMAX; idx < p.M * units; idx += FUSED_THREADS) {
            const int tok = idx / units, u = idx - tok * units;
            const int k0 = k_begin + u * 16;
            if (k0 < p.K) {
                Raw16<HALF> r;
                load_raw<HALF>(A + (size_t)tok * p.K, k0, p.K, vec, r);
                atomicMax(&s_max[tok], raw_maxbits<HALF>(r));
            }
        }
        __syncthreads();
        if (S > 1) {
            // every rank sends its slice maxima to every rank (itself included); a rank goes on as soon as
            // the S * TC words it expects have landed -- no cluster-wide barrier on the critical path
            cluster_wait();
            for (int i = tid; i < S * TC; i += FUSED_THREADS) {
                const int r = i / TC, t = i - r * TC;
                st_async_u32(map_to_cta(smem_u32(&inbox_max[rank * TC + t]), (uint32_t)r), s_max[t], map_to_cta(smem_u32(&full[0]), (uint32_t)r));
            }
            if (!mbar_wait(&full[0], 0, deadline)) s_flags[1] = 1;   // (every thread polls: electing one lane per warp measured 8 % slower)
        }
    }
    if (tid < TC) {
        uint32_t bits = 0;
        int bad = 0;
        float maximum;
        if (p.rowmax_in != nullptr) {
            bits = tid < p.M ? p.rowmax_in[tid] : 0u;
            bad = bits >= 0x7f800000u ? 2 : 0;
            maximum = __uint_as_float(bits);
        } else {
            if (S > 1) for (int r = 0; r < S; ++r) bits = max(bits, inbox_max[r * TC + tid]);
            else bits = s_max[tid];
            if constexpr (HALF) { bad = bits >= 0x7c00u ? 1 : 0; maximum = __half2float(__ushort_as_half((uint16_t)bits)); }
            else { bad = bits >= 0x7f800000u ? 1 : 0; maximum = __uint_as_float(bits); }
        }
        float s, inv;
        scale_from_max(maximum, bad != 0, s, inv);
        s_scale[tid] = s;
        s_inv[tid] = inv;
        if (bad) atomicOr(&s_flags[0], bad);
        if (blockIdx.x == 0 && rank == 0 && tid < p.M && p.scales_out) p.scales_out[tid] = s;
    }
    __syncthreads();
    if (trace) trace[3] = (unsigned long long)(clock64() - c_start);
    const int verdict = s_flags[0];   // identical in every CTA: all of them saw the whole rows
    // partial sums this rank will receive: its share of the channels, every token, from every rank
    const int Qq = p.epi == EPI_SWIGLU ? 16 : 32;
    const int my_quads = ((rank + 1) * Qq) / S - (rank * Qq) / S;
    if (tid == 0 && S > 1 && !verdict)
        for (int i = 0; i < ntile; ++i)
            mbar_arrive_expect_tx(&full[3 + i], (uint32_t)(S * TC * my_quads * 4 * (p.epi == EPI_SWIGLU ? 2 : 1) * 4));

    // ---- 2. quantise the slice into shared memory: xs[unit][token][16 B]
    if (!verdict) {
#pragma unroll
        for (int it = 0; it < UMAX; ++it) {
            const int idx = tid + FUSED_THREADS * it;
            if (idx < items) {
                const int tok = pos_tok[it], u = pos_u[it];
                const uint4 q = quantize_unit<HALF>(kept[it], s_inv[tok], k_begin + u * 16, p.K);   // padding rows hold zeros
                reinterpret_cast<uint4*>(xs)[(size_t)u * TC + tok] = q;
                if (p.codes_out && blockIdx.x == 0) reinterpret_cast<uint4*>(p.codes_out)[((size_t)kb0 * 8 + u) * TC + tok] = q;
            }
        }
        for (int idx = tid + FUSED_THREADS * UMAX; idx < items; idx += FUSED_THREADS) {
            const int tok = idx / units, u = idx - tok * units;
            const int k0 = k_begin + u * 16;
            uint4 q = make_uint4(0u, 0u, 0u, 0u);
            if (tok < p.M && k0 < p.K) {
                Raw16<HALF> r;
                load_raw<HALF>(A + (size_t)tok * p.K, k0, p.K, vec, r);
                q = quantize_unit<HALF>(r, s_inv[tok], k0, p.K);
            }
            reinterpret_cast<uint4*>(xs)[(size_t)u * TC + tok] = q;
            if (p.codes_out && blockIdx.x == 0) reinterpret_cast<uint4*>(p.codes_out)[((size_t)kb0 * 8 + u) * TC + tok] = q;
        }
    }
    __syncthreads();

    if (trace) trace[4] = (unsigned long long)(clock64() - c_start);
    const int g8 = lane >> 2, t4 = lane & 3;
    const int wgroup = warp >> 1, mtile = warp & 1;
    // Channel ownership in quads of four: rank r finishes quads [r*Q/S, (r+1)*Q/S) of the CTA's
    // Q quads (gate quads for SwiGLU, whose up partner travels with it); W = widest share.
    const int Q = swiglu ? 16 : 32;
    const int q_first = (rank * Q) / S, q_count = ((rank + 1) * Q) / S - q_first;
    const int QW = (Q + S - 1) / S;                // quads per inbox row half
    const int W = (swiglu ? 2 : 1) * QW * 4;       // words per token per source rank
    if (S > 1 && p.rowmax_in != nullptr) cluster_wait();

    // The CTA's column tiles one after the other: the quantised slice is shared, the second tile's weights
    // are requested into the same shared memory as soon as the first tile's contraction has read them, and
    // arrive while the first tile's partial sums are exchanged and finished.
    for (int ti = 0; ti < ntile; ++ti) {
    if (verdict && ti > 0) break;            // rejected input: nothing was requested for the second tile
    const int tile = tile_first + ti;
    int32_t* const inbox_sum = inbox_all + (size_t)ti * TC * 192;
    // ---- 3. contraction: warp w owns the m16 tile (w & 1) of weight group (w >> 1)
    int acc[NT][4], acc2[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[j][e] = 0; acc2[j][e] = 0; }
    // The copies have to land before this CTA may leave, whatever the verdict.
    if (nkb > 0 && !mbar_wait(&full[1 + ti], 0, deadline)) s_flags[1] = 1;
    for (int s = 0; s < (verdict ? 0 : nkb); ++s) {
        const uint32_t* const wbase = reinterpret_cast<const uint32_t*>(wst + ((size_t)wgroup * nkb + s) * 2048 + (mtile * 16 + g8) * 16) + t4;
        const uint32_t* const xbase = reinterpret_cast<const uint32_t*>(xs + (size_t)s * TC * 128 + g8 * 16) + t4;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t w0 = wbase[c * 128];
            const uint32_t w1 = wbase[c * 128 + 32];
            const uint32_t a0 = (w0 << 4) & 0xF0F0F0F0u, a1 = (w1 << 4) & 0xF0F0F0F0u;
            const uint32_t a2 = w0 & 0xF0F0F0F0u, a3 = w1 & 0xF0F0F0F0u;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint32_t b0 = xbase[((2 * c) * TC + 8 * j) * 4];
                const uint32_t b1 = xbase[((2 * c + 1) * TC + 8 * j) * 4];
                // two accumulator sets halve the chain of dependent MMAs (integer sums: any order is exact)
                if (c & 1) mma_s8(acc2[j], a0, a1, a2, a3, b0, b1);
                else mma_s8(acc[j], a0, a1, a2, a3, b0, b1);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] += acc2[j][e];

    if (ti + 1 < ntile && !verdict) {
        // every warp has read this tile's weights: fetch the next tile's into the same place
        __syncthreads();
        if (tid == 0 && nkb > 0) mbar_arrive_expect_tx(&full[2 + ti], (uint32_t)nkb * 8192u);
        if (tid < 4 && nkb > 0) request_weights(tile + 1, &full[2 + ti]);
    }
    if (trace) trace[5] = (unsigned long long)(clock64() - c_start);
    // ---- 4. partial sums to the rank that owns the channel: inbox_sum[source][token][W]
    if (!verdict) {
        // A thread's fragment holds two channels (rows g8 and g8 + 8 of its m16 tile); who finishes each of them and
        // where it lands there is worked out once per channel, with a shift for the quad count (16 or 32).
        int owner2[2], local2[2];
        uint32_t dst_bar[2];
        const int lq = swiglu ? 4 : 5;                                  // log2(Q)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int ch = wgroup * 32 + mtile * 16 + g8 + h * 8;
            const int c = swiglu ? (ch & 63) : ch;
            owner2[h] = ((((c >> 2) + 1) * S + Q - 1) >> lq) - 1;
            local2[h] = c - ((owner2[h] * Q) / S) * 4 + ((swiglu && ch >= 64) ? QW * 4 : 0);
            dst_bar[h] = S > 1 ? map_to_cta(smem_u32(&full[3 + ti]), (uint32_t)owner2[h]) : 0u;
        }
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const int tok = 8 * j + 2 * t4 + (e & 1);
                const int word = (rank * TC + tok) * W + local2[h];
                const int value = acc[j][e] >> 4;                       // exact: sums are multiples of 16
                if (S > 1) st_async_u32(map_to_cta(smem_u32(&inbox_sum[word]), (uint32_t)owner2[h]), (uint32_t)value, dst_bar[h]);
                else inbox_sum[word] = value;
            }
    }
    if (S > 1) {
        if (!verdict && !mbar_wait(&full[3 + ti], 0, deadline)) s_flags[1] = 1;
    } else __syncthreads();
    if (trace) trace[6] = (unsigned long long)(clock64() - c_start);

    // ---- 5. finish the channels this rank owns
    if (!verdict) {
        const int IPT = q_count;
        const int out_items = TC * IPT;
        for (int base = 0; base < out_items; base += FUSED_THREADS) {
            const int i = base + tid;
            const bool active = i < out_items;
            const int tok = active ? i / IPT : 0, c4 = active ? i - tok * IPT : 0;
            int v[4] = {0, 0, 0, 0}, u[4] = {0, 0, 0, 0};
            if (active) {
                for (int q = 0; q < S; ++q) {
                    const int4 a = *reinterpret_cast<const int4*>(inbox_sum + (q * TC + tok) * W + c4 * 4);
                    v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
                    if (swiglu) {
                        const int4 b = *reinterpret_cast<const int4*>(inbox_sum + (q * TC + tok) * W + QW * 4 + c4 * 4);
                        u[0] += b.x; u[1] += b.y; u[2] += b.z; u[3] += b.w;
                    }
                }
            }
            const bool row_ok = active && tok < p.M;
            const float sx = s_scale[tok];
            if (!swiglu) {
                const int n = tile * TILE_N + (q_first + c4) * 4;
                if (row_ok && n < p.N) {
                    const int valid = min(4, p.N - n);
                    if (p.epi == EPI_I32) {
                        store4_i32(reinterpret_cast<int*>(p.out) + (size_t)tok * p.N + n, v, valid);
                    } else {
                        float y[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) y[e] = dequant(v[e], sx, s_sw[(q_first + c4) * 4 + e]);
                        if (p.epi == EPI_F32) store4_f32(reinterpret_cast<float*>(p.out) + (size_t)tok * p.N + n, y, valid);
                        else store4_f16(reinterpret_cast<__half*>(p.out) + (size_t)tok * p.N + n, y, valid);
                    }
                }
            } else {
                const int f = tile * 64 + (q_first + c4) * 4;
                if (row_ok && f < p.F) {
                    float y[4];
                    uint32_t mx = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float g = dequant(v[e], sx, s_sw[(q_first + c4) * 4 + e]);
                        const float up = dequant(u[e], sx, s_sw[64 + (q_first + c4) * 4 + e]);
                        y[e] = __fmul_rn(silu_poly(g), up);
                        mx = max(mx, __float_as_uint(y[e]) & 0x7fffffffu);
                    }
                    store4_f32(reinterpret_cast<float*>(p.out) + (size_t)tok * p.F + f, y, 4);
                    if (p.rowmax_out && mx) atomicMax(&s_outmax[tok], mx);
                }
            }
        }
    }
    if (ti + 1 < ntile) {
        __syncthreads();                      // the channel scales of this tile have been used by everybody
        stage_channel_scales(tile + 1);
        __syncthreads();
    }
    }   // tiles of this CTA
    if (!verdict && swiglu && p.rowmax_out) {
        __syncthreads();
        if (tid < p.M && s_outmax[tid]) atomicMax(&p.rowmax_out[tid], s_outmax[tid]);
    }

    // ---- bookkeeping by one thread per CTA
    if (trace) trace[7] = global_ns();
    if (tid == 0) {
        if (s_flags[1]) *reinterpret_cast<volatile int*>(&p.status->device_error) = 1;   // (plain store: may be page-locked host memory)
        if (blockIdx.x == 0 && rank == 0) p.status->bad_input = verdict;
        if (p.rowmax_in != nullptr) {
            // Every CTA has read the row maxima by now; the last one to get here clears
            // them for the next SwiGLU epilogue.  The ticket counter wraps by itself.
            __threadfence();
            const unsigned total = gridDim.x * gridDim.y;
            if (atomicInc(&p.status->done, total - 1u) == total - 1u)
                for (int t = 0; t < p.M; ++t) p.rowmax_in[t] = 0u;
        }
    }
}

size_t gemm_fused_smem_bytes(int tokens_per_cta, int stages, int tiles_per_cta) { return fused_smem_bytes(tokens_per_cta, stages, tiles_per_cta); }

template <int NT, bool HALF>
static cudaError_t launch_fused_inst(const FusedParams& p, cudaStream_t stream, bool pdl)
{
    constexpr int TC = 8 * NT;
    auto kernel = gemm_fused_kernel<NT, HALF>;
    static PerDeviceOnce configured;
    int configured_device = -1;
    if (configured.needed(configured_device)) {
        const size_t most = fused_smem_bytes(TC, FUSED_MAX_STAGES, 2) < FUSED_SMEM_LIMIT ? fused_smem_bytes(TC, FUSED_MAX_STAGES, 2) : FUSED_SMEM_LIMIT;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
        if (e != cudaSuccess) return e;
        configured.mark(configured_device);
    }
    const int tiles = p.epi == EPI_SWIGLU ? (p.F + 63) / 64 : (p.N + TILE_N - 1) / TILE_N;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((tiles + p.tiles_per_cta - 1) / p.tiles_per_cta), (unsigned)p.split, 1);
    cfg.blockDim = dim3(FUSED_THREADS);
    cfg.dynamicSmemBytes = fused_smem_bytes(TC, p.stages, p.tiles_per_cta);
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

cudaError_t launch_gemm_fused(const FusedParams& p, int tokens_per_cta, cudaStream_t stream, bool pdl)
{
    if (p.split < 1 || p.split > 8 || p.M > tokens_per_cta || p.tiles_per_cta < 1 || p.tiles_per_cta > 2 ||
        fused_smem_bytes(tokens_per_cta, p.stages, p.tiles_per_cta) > FUSED_SMEM_LIMIT ||
        p.stages > FUSED_MAX_STAGES || p.stages * p.split < p.KB || (long long)p.KB * KBLOCK > 131072)
        return cudaErrorInvalidValue;
    switch (tokens_per_cta) {
    case 8: return p.half ? launch_fused_inst<1, true>(p, stream, pdl) : launch_fused_inst<1, false>(p, stream, pdl);
    case 16: return p.half ? launch_fused_inst<2, true>(p, stream, pdl) : launch_fused_inst<2, false>(p, stream, pdl);
    case 32: return p.half ? launch_fused_inst<4, true>(p, stream, pdl) : launch_fused_inst<4, false>(p, stream, pdl);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace rkb200
