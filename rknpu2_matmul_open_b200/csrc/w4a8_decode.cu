// w4a8_decode.cu -- single-kernel W4A8 linear for up to eight tokens (decode) on sm_100a.
//
// One launch does what the reference does in three stages (scan + quantise, src/
// rk_npu_w4a8_quant.cpp:52-135; contraction; reconstruct + dequantise / SwiGLU, src/
// rk_npu_w4a8_output.cpp:35-161, src/rk_npu_w4a8_swiglu.cpp:12-91).  The launch is HBM-bound on its
// weight stream, and in a chain of dependent linears what is not hidden behind that stream is the
// latency between "the activations exist" and "the outputs are stored".  The kernel is built to keep
// that chain short:
//
//   * A CTA owns whole output channels: 32-channel weight groups (a gate group and its up partner for
//     SwiGLU) over ALL of K, dealt round-robin to the CTAs.  Nothing is summed across CTAs; the K range
//     is split over the CTA's own eight contraction warps and summed through its shared memory.
//   * A ninth warp streams the CTA's weights through a ring of 32 KB stages with bulk async copies.
//     Weights never change, so everything the ring holds is requested BEFORE the programmatic
//     dependency wait and arrives while the launch in front is still running.
//   * Quantising M x K activations costs about eleven instructions per element, more than the whole
//     contraction when every CTA does all of it, so the CTAs of a cluster share it: each scans the full
//     rows of its tokens for the maximum (or its tokens' scale comes from collected row maxima),
//     quantises its share into its own shared memory -- plain int8 rows, one per token -- and hands the
//     share to every other member with ONE bulk copy per member (shared memory to the peer's shared
//     memory, counted in bytes on the peer's mbarrier).  That is the only exchange of the launch; small
//     problems run without a cluster and quantise locally.
//   * The contraction uses mma.sync m16n8k32 (16 channels x 8 token columns) for every token count: on
//     this GPU it needs fewer issue slots per weight byte than integer dot products even for one token.
//     Full 32 KB stages run a loop without per-load predicates; only a K tail takes the guarded form.
//
// Integer sums are exact in any order, so the warp split and the four accumulator sets per warp do not
// change results.
#include "w4a8_device.h"
#include "w4a8_math.cuh"
#include "w4a8_ptx.cuh"

namespace rkb200 {

constexpr int DEC_WARPS = 8;                        // contraction warps
constexpr int DEC_THREADS = (DEC_WARPS + 1) * 32;   // + the copy warp
constexpr int DEC_STAGE_CHUNKS = 64;                // 32-element chunks (2048 reduction elements) of one weight group per stage: 32 KB
constexpr int DEC_STAGE_BYTES = DEC_STAGE_CHUNKS * 512;
constexpr int DEC_ROW_PAD = 16;                     // bytes behind a token's code row: rows of different tokens start in different banks
constexpr size_t DEC_SMEM_LIMIT = 227 * 1024;

__host__ __device__ constexpr int dec_token_slots(int M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8; }
__host__ __device__ constexpr size_t dec_fixed_bytes(int M, int KB, bool swiglu)
{
    return (size_t)dec_token_slots(M) * (KB * KBLOCK + DEC_ROW_PAD)   // activation codes of all of K, one row per token
           + (size_t)DEC_WARPS * (swiglu ? 64 : 32) * 8 * 4           // per-warp partial sums
           + 96 + 8;                                                  // row maxima, scale words, inverse scales; + barriers below
}
__host__ __device__ constexpr size_t dec_smem_bytes(int M, int KB, bool swiglu, int ring)
{
    return dec_fixed_bytes(M, KB, swiglu) + (size_t)ring * DEC_STAGE_BYTES + (size_t)(2 * ring + 1) * 8;
}

// Bulk copy from this CTA's shared memory into a cluster member's, counted in bytes on a barrier there.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_s2s(uint32_t remote_dst, uint32_t local_src, uint32_t bytes, uint32_t remote_bar)
{
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(remote_dst),
                 "r"(local_src), "r"(bytes), "r"(remote_bar)
                 : "memory");
}
// Wait of a whole warp on an mbarrier phase.  Fast path: the phase is already complete (weights are normally
// requested long before they are needed) and one test by every lane both sees that and gives each lane its
// acquire; otherwise one lane polls with the bounded wait and the others follow it.
// The time limit starts the first time a warp really has to wait (reading the global timer costs a few hundred cycles,
// too many for the path behind the dependency, and a limit taken in front of the dependency wait would charge the
// launch in front to this one): `deadline_ns` is 0 until then.
__device__ __forceinline__ bool mbar_wait_all_lanes(uint64_t* bar, uint32_t parity, unsigned long long& deadline_ns, unsigned long long timeout_ns)
{
    if (__all_sync(0xffffffffu, mbar_test(bar, parity))) return true;
    if (deadline_ns == 0) deadline_ns = global_ns() + timeout_ns;
    return mbar_wait_warp(bar, parity, deadline_ns);
}
__device__ __forceinline__ void bar_sync_contraction() { asm volatile("bar.sync 1, %0;" ::"n"(DEC_WARPS * 32) : "memory"); }

// Partial-sum scratch index: [warp][row][token], the token position XOR-ed with row bits so that both the
// fragment-shaped writes and the (token, row)-shaped reads are free of bank conflicts.
__device__ __forceinline__ int red_index(int warp, int rows, int row, int tok)
{
    return (warp * rows + row) * 8 + (tok ^ ((row >> 2) & 7));
}

// Rows longer than a thread's register budget (more than UMAX units per thread): the remaining units are scanned and
// later quantised by these two routines, from memory.  Out of line: the shapes the kernel is tuned for never get here,
// and inlined they were a fifth of the kernel's instruction stream.
template <bool HALF>
static __device__ __noinline__ void scan_rest(const typename ActType<HALF>::type* A, int K, bool vec, int first, int scan_items, int TQ, int su0,
                                              int sn, int t0, int M, uint32_t* s_max)
{
    for (int idx = first; idx < scan_items; idx += DEC_WARPS * 32) {
        const int tl = TQ > 1 ? idx / sn : 0, u = su0 + idx - tl * sn;
        if (t0 + tl < M && u * 16 < K) {
            Raw16<HALF> r;
            load_raw<HALF>(A + (size_t)(t0 + tl) * K, u * 16, K, vec, r);
            atomicMax(&s_max[tl], raw_maxbits<HALF>(r));
        }
    }
}
template <bool HALF>
static __device__ __noinline__ void quantize_rest(const typename ActType<HALF>::type* A, int K, bool vec, int first, int scan_items, int TQ,
                                                  int su0, int sn, int t0, int M, int pu0, int pu1, const float* s_inv, uint8_t* xs,
                                                  int row_bytes, uint8_t* codes_out)
{
    for (int idx = first; idx < scan_items; idx += DEC_WARPS * 32) {
        const int tl = TQ > 1 ? idx / sn : 0, u = su0 + idx - tl * sn;
        if (t0 + tl < M && u >= pu0 && u < pu1) {
            Raw16<HALF> r;
            load_raw<HALF>(A + (size_t)(t0 + tl) * K, u * 16, K, vec, r);
            const uint4 q = quantize_unit<HALF>(r, s_inv[tl], u * 16, K);
            *reinterpret_cast<uint4*>(xs + (size_t)(t0 + tl) * row_bytes + (size_t)u * 16) = q;
            if (codes_out) reinterpret_cast<uint4*>(codes_out)[(size_t)u * 8 + t0 + tl] = q;
        }
    }
}

// One CTA of one linear: `cta` of `nctas` (the kernels below map the grid onto one or several linears).
// The CTA's path between "the activations exist" and "the outputs are stored" is a chain of short phases run by
// nine warps, so it is bound by instruction latency and issue slots, not memory: the code avoids integer
// divisions, computes a token's scale once, and gives every warp four independent accumulator sets per stage.
template <bool HALF, bool TRACE>
__device__ __forceinline__ void decode_cta(const DecodeParams& p, const unsigned cta, const unsigned nctas)
{
    using AT = typename ActType<HALF>::type;
    extern __shared__ __align__(128) uint8_t smem[];
    const int R = p.ring;
    const int M = p.M;
    const int Mc = dec_token_slots(M);
    const int Kp = p.KB * KBLOCK, U = Kp / 16, KC = p.KB * 4;
    const int row_bytes = Kp + DEC_ROW_PAD;
    const bool swiglu = p.epi == EPI_SWIGLU;
    const int rows = swiglu ? 64 : 32;
    uint8_t* const ring = smem;
    uint8_t* const xs = ring + (size_t)R * DEC_STAGE_BYTES;                     // codes: [token][Kp + pad] int8
    int* const red = reinterpret_cast<int*>(xs + (size_t)Mc * row_bytes);
    uint32_t* const s_max = reinterpret_cast<uint32_t*>(red + DEC_WARPS * rows * 8);   // [8] row maxima of this CTA's tokens
    uint32_t* const s_scale = s_max + 8;                                         // [8] scale bits per token (or 0xFFFFFFF0 | verdict)
    float* const s_inv = reinterpret_cast<float*>(s_scale + 8);                  // [8] inverse scales of this CTA's tokens
    uint64_t* const full = reinterpret_cast<uint64_t*>(s_inv + 8 + 2);
    uint64_t* const empty = full + R;
    uint64_t* const code_bar = empty + R;

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.cluster, rank = S > 1 ? (int)(cta % (unsigned)S) : 0;
    const int ncta = (int)nctas;
    const int items = swiglu ? p.F / GROUP : (p.N + GROUP - 1) / GROUP;
    const int gpi = swiglu ? 2 : 1;                                              // weight groups per item
    const int my_items = (int)cta < items ? (items - 1 - (int)cta) / ncta + 1 : 0;
    unsigned long long* const trace = (TRACE && p.trace && tid == 0) ? p.trace + (size_t)cta * 8 : nullptr;
    long long c_start = 0;
    if (TRACE) { c_start = clock64(); if (trace) trace[0] = global_ns(); }
    auto stamp = [&](int slot) { if (TRACE && trace && cta == 0) p.trace[8 * 4096 + slot] = (unsigned long long)(clock64() - c_start); };

    // ---- this CTA's share of the quantisation.  Mc >= S: whole rows of TQ tokens; else one token's
    // K range is split over P CTAs, each of which still scans the whole row for the maximum.
    int TQ, P, t0, part;
    if (Mc >= S) { TQ = Mc / S; P = 1; t0 = rank * TQ; part = 0; }
    else { TQ = 1; P = S / Mc; t0 = rank / P; part = rank - t0 * P; }
    const int pu0 = (int)((long long)U * part / P), pu1 = (int)((long long)U * (part + 1) / P);
    // the bytes of the code rows this CTA produces (contiguous: whole rows, or a piece of one row)
    const uint32_t share_off = (uint32_t)t0 * (uint32_t)row_bytes + (uint32_t)pu0 * 16u;
    const uint32_t share_bytes = P == 1 ? (uint32_t)TQ * (uint32_t)row_bytes : (uint32_t)(pu1 - pu0) * 16u;

    if (tid == 0) {
        for (int i = 0; i < R; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], DEC_WARPS); }
        mbar_init(code_bar, 1);
        mbar_fence_init();
        if (S > 1) {
            // what the other members send: every token's row (all of them when rows are split) minus this CTA's own share,
            // plus one scale word per live token
            const uint32_t all = P == 1 ? (uint32_t)Mc * (uint32_t)row_bytes : (uint32_t)Mc * (uint32_t)U * 16u;
            mbar_arrive_expect_tx(code_bar, all - share_bytes + (uint32_t)M * 4u);
        }
    }
    if (tid < 8) s_max[tid] = 0u;
    __syncthreads();
    if (S > 1) cluster_arrive();   // every member's barriers exist once the matching wait returns

    // ------------------------------------------------------------------ copy warp
    if (warp == DEC_WARPS) {
        if (S > 1) cluster_wait();
        if (lane == 0) {
            unsigned long long deadline = ~0ull;
            int slot = 0, issued = 0;
            uint32_t turn = 0;                      // how often the ring has wrapped
            for (int j = 0; j < my_items; ++j) {
                const int item = (int)cta + j * ncta;
                for (int g = 0; g < gpi; ++g) {
                    const size_t group = (size_t)(g == 0 ? item : p.F / GROUP + item);
                    for (int c0 = 0; c0 < KC; c0 += DEC_STAGE_CHUNKS, ++issued) {
                        if (issued >= R) {
                            if (issued == R) {      // from here on a slot must be handed back first, which cannot happen before the dependency
                                pdl_wait();
                                deadline = global_ns() + p.timeout_ns;
                            }
                            if (!mbar_wait(&empty[slot], (turn - 1u) & 1u, deadline)) {
                                *reinterpret_cast<volatile int*>(&p.status->device_error) = 1;   // (a plain store: the block may be page-locked host memory)
                                return;
                            }
                        }
                        const uint32_t bytes = (uint32_t)min(DEC_STAGE_CHUNKS, KC - c0) * 512u;
                        // (test hook: 16 bytes that no copy brings keep the first barrier open until the wait gives up;
                        // every real copy still lands)
                        mbar_arrive_expect_tx(&full[slot], bytes + ((p.starve && issued == 0) ? 16u : 0u));
                        bulk_g2s(ring + (size_t)slot * DEC_STAGE_BYTES, p.Wp + (group * KC + c0) * 512, bytes, &full[slot]);
                        if (++slot == R) { slot = 0; ++turn; }
                    }
                }
            }
        }
        return;
    }

    // ------------------------------------------------------------------ contraction warps
    // channel scales of an item's outputs (constants: the first item's are read before the dependency)
    float sw_a = 0.f, sw_b = 0.f;
    auto load_channel_scales = [&](int item) {
        const int n = item * GROUP + lane;
        sw_a = n < p.NG * GROUP ? p.sw[n] : 0.f;
        if (swiglu) sw_b = p.sw[p.F + n];
    };
    if (my_items > 0) load_channel_scales((int)cta);

    const bool no_scan = p.rowmax_in != nullptr;
    const int su0 = no_scan ? pu0 : 0, sn = (no_scan ? pu1 : U) - su0;
    const int scan_items = TQ * sn;
    // item index -> (local token, unit); no division in the common one-token case
    auto locate = [&](int idx, int& tl, int& u) {
        tl = 0;
        if (TQ > 1) tl = idx / sn;
        u = su0 + idx - tl * sn;
    };
    const AT* A = reinterpret_cast<const AT*>(p.A);
    const bool vec = (reinterpret_cast<uintptr_t>(A) & 15u) == 0 && (p.K % (HALF ? 8 : 4)) == 0;
    constexpr int UMAX = HALF ? 3 : 2;     // units a thread keeps in registers between the scan and the quantisation
    constexpr int CT = DEC_WARPS * 32;
    // Everything that does not need the activations is settled before the wait: where this thread's units lie (no
    // division behind the dependency).
    int pos_tl[UMAX], pos_u[UMAX];
    bool pos_live[UMAX];
#pragma unroll
    for (int it = 0; it < UMAX; ++it) {
        const int idx = tid + CT * it;
        pos_tl[it] = 0;
        pos_u[it] = 0;
        if (idx < scan_items) locate(idx, pos_tl[it], pos_u[it]);
        pos_live[it] = idx < scan_items && t0 + pos_tl[it] < M;
        // The unit this thread will read, pulled towards L2 while the launch in front still runs.  A prefetch is only
        // a hint: the L2 is the point of coherence, so whatever the producer still writes is what the load sees.
        if (pos_live[it] && pos_u[it] * 16 < p.K)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(A) + ((size_t)(t0 + pos_tl[it]) * p.K + (size_t)pos_u[it] * 16) * sizeof(AT)));
    }
    unsigned long long deadline = 0;   // set by the first wait that does not find its barrier complete
    if (TRACE && trace) trace[1] = (unsigned long long)(clock64() - c_start);
    // The producer of A (and of the collected row maxima) has finished once the dependency wait returns.  One warp
    // executes it; the others block at the hardware barrier behind it, where they take no issue slots from the
    // launch in front, whose CTAs share this SM while it finishes.
    if (warp == 0) pdl_wait();
    bar_sync_contraction();
    if (TRACE && trace) trace[2] = (unsigned long long)(clock64() - c_start);

    Raw16<HALF> kept[UMAX];
    // every load is issued before anything waits for one: a round trip to L2 costs more than the rest of the scan
#pragma unroll
    for (int it = 0; it < UMAX; ++it) {
#pragma unroll
        for (int i = 0; i < (HALF ? 8 : 16); ++i) kept[it].w[i] = 0u;
        if (pos_live[it] && pos_u[it] * 16 < p.K) load_raw<HALF>(A + (size_t)(t0 + pos_tl[it]) * p.K, pos_u[it] * 16, p.K, vec, kept[it]);
    }
    uint32_t collected = 0;                   // no_scan: this thread's token's collected maximum
    if (no_scan && tid < TQ && t0 + tid < M) collected = p.rowmax_in[t0 + tid];
    stamp(64);
    if (!no_scan) {
#pragma unroll
        for (int it = 0; it < UMAX; ++it) {
            const int tl = pos_tl[it];
            const uint32_t bits = raw_maxbits<HALF>(kept[it]);    // units never loaded hold zeros
            // a warp whose 32 units belong to one token reduces first and issues a single shared atomic; one code
            // path for both cases (every warp-wide operation is executed by all 32 lanes, none behind a lane condition)
            const int tl0 = __shfl_sync(0xffffffffu, tl, 0);
            const bool uniform = TQ == 1 || __all_sync(0xffffffffu, tl == tl0);
            const uint32_t reduced = __reduce_max_sync(0xffffffffu, bits);
            const uint32_t mine = uniform ? reduced : bits;
            if ((!uniform || lane == 0) && mine) atomicMax(&s_max[uniform ? tl0 : tl], mine);
        }
        if (scan_items > CT * UMAX) scan_rest<HALF>(A, p.K, vec, tid + CT * UMAX, scan_items, TQ, su0, sn, t0, M, s_max);
        stamp(65);
        bar_sync_contraction();
    }
    const bool first_cluster = (int)cta < S;
    const uint32_t xs_base = smem_u32(xs), bar_base = smem_u32(code_bar);
    // One thread per token derives its scale -- s = max(maximum / 127, FLT_MIN), 1 for a zero row; inverse = 1 / s, two
    // IEEE divisions -- once, and (from the CTA that holds the token's first K part) sends it to every cluster member.
    if (S > 1) cluster_wait();
    if (tid < TQ) {
        const int tok = t0 + tid;
        int bad = 0;
        float maximum = 0.f, sc = 1.f, inv = 1.f;
        if (tok < M) {
            if (no_scan) {
                bad = collected >= 0x7f800000u ? 2 : 0;
                maximum = __uint_as_float(collected);
            } else {
                const uint32_t bits = s_max[tid];
                if constexpr (HALF) { bad = bits >= 0x7c00u ? 1 : 0; maximum = __half2float(__ushort_as_half((uint16_t)bits)); }
                else { bad = bits >= 0x7f800000u ? 1 : 0; maximum = __uint_as_float(bits); }
            }
            scale_from_max(maximum, bad != 0, sc, inv);
        }
        s_inv[tid] = inv;
        if (part == 0 && tok < M) {
            const uint32_t word = bad ? (0xFFFFFFF0u | (uint32_t)bad) : __float_as_uint(sc);
            if (S > 1) {
                for (int d = 0; d < S; ++d)
                    st_async_u32(map_to_cta(smem_u32(&s_scale[tok]), (uint32_t)d), word, map_to_cta(bar_base, (uint32_t)d));
            } else s_scale[tok] = word;
            if (first_cluster && p.scales_out) p.scales_out[tok] = sc;
        }
    }
    bar_sync_contraction();
    stamp(66);
    // ---- quantise this CTA's share into its own code rows
    auto keep_code = [&](int tok, int u, const uint4& q) {
        *reinterpret_cast<uint4*>(xs + (size_t)tok * row_bytes + (size_t)u * 16) = q;
        if (p.codes_out && first_cluster) reinterpret_cast<uint4*>(p.codes_out)[(size_t)u * 8 + tok] = q;
    };
#pragma unroll
    for (int it = 0; it < UMAX; ++it) {
        const int tl = pos_tl[it], u = pos_u[it];
        if (pos_live[it] && u >= pu0 && u < pu1) keep_code(t0 + tl, u, quantize_unit<HALF>(kept[it], s_inv[tl], u * 16, p.K));
    }
    if (scan_items > CT * UMAX)
        quantize_rest<HALF>(A, p.K, vec, tid + CT * UMAX, scan_items, TQ, su0, sn, t0, M, pu0, pu1, s_inv, xs, row_bytes,
                            (p.codes_out && first_cluster) ? p.codes_out : nullptr);
    stamp(67);
    bool failed = false;
    if (S > 1) {
        // ---- hand the share to every other member: one bulk copy each, issued by one thread per destination once
        // every thread's stores are visible to the copy engine
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        bar_sync_contraction();
        if (tid < S && tid != rank)
            bulk_s2s(map_to_cta(xs_base + share_off, (uint32_t)tid), xs_base + share_off, share_bytes, map_to_cta(bar_base, (uint32_t)tid));
        if (TRACE && trace) trace[3] = (unsigned long long)(clock64() - c_start);
        // (every thread polls this one: on the critical path an elected lane per warp wakes its warp later -- the same
        // change cost the split-K kernel 8 %)
        if (!mbar_test(code_bar, 0)) {
            if (deadline == 0) deadline = global_ns() + p.timeout_ns;
            if (!mbar_wait(code_bar, 0, deadline)) failed = true;
        }
        failed = __any_sync(0xffffffffu, failed);
    } else {
        if (TRACE && trace) trace[3] = (unsigned long long)(clock64() - c_start);
        bar_sync_contraction();
    }
    if (TRACE && trace) trace[4] = (unsigned long long)(clock64() - c_start);
    int verdict = 0;
#pragma unroll
    for (int t = 0; t < 8; ++t) {            // eight independent broadcast reads, not a chain of them
        const uint32_t w = t < M ? s_scale[t] : 0u;
        if (w >= 0xFFFFFFF0u) verdict |= (int)(w & 0xFu);
    }

    // ---- contraction: warp w takes the chunks w, w + 8, ... of every stage, all 32 (64) channels
    const int g8 = lane >> 2, t4 = lane & 3;
    const bool col_live = g8 < M;
    const int tok_out = tid >> 5;                         // epilogue: this thread's token; its channel is `lane`
    const float sx = (tok_out < M && !verdict) ? __uint_as_float(s_scale[tok_out]) : 0.f;
    const bool compute = !verdict;
    // this lane's two words of a chunk: token g8's codes k = 32c + 4 t4 .. and k = 32c + 16 + 4 t4 ..
    const uint32_t* const xlane = reinterpret_cast<const uint32_t*>(xs + (size_t)(col_live ? g8 : 0) * row_bytes) + t4;
    uint32_t run_max = 0;
    int slot = 0, stage_no = 0;
    uint32_t parity = 0;
    // hands the stage back and moves on to the next ring slot
    auto release_stage = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
        if (++slot == R) { slot = 0; parity ^= 1u; }
        ++stage_no;
    };
    auto acquire_stage = [&]() {
        if (TRACE && stage_no < 8) stamp(2 * stage_no);
        if (!mbar_wait_all_lanes(&full[slot], parity, deadline, p.timeout_ns)) failed = true;
        if (TRACE && stage_no < 8) stamp(2 * stage_no + 1);
    };
    for (int j = 0; j < my_items; ++j) {
        const int item = (int)cta + j * ncta;
        // One pass per weight group of the item (gate, then up for SwiGLU): a run-time loop, so that the stage loop
        // exists once in the instruction stream; a pass leaves its partial sums in the scratch rows of its group.
#pragma unroll 1
        for (int g = 0; g < gpi; ++g) {
            // four accumulator sets: four of a warp's chunks of a stage are independent MMAs, so their loads and the
            // latency of the MMAs overlap
            int a[4][2][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int m = 0; m < 2; ++m)
#pragma unroll
                    for (int e = 0; e < 4; ++e) a[i][m][e] = 0;
            for (int c0 = 0; c0 < KC; c0 += DEC_STAGE_CHUNKS) {
                acquire_stage();
                if (compute && !failed) {
                    const int nch = min(DEC_STAGE_CHUNKS, KC - c0);
                    const uint32_t* const wslot = reinterpret_cast<const uint32_t*>(ring + (size_t)slot * DEC_STAGE_BYTES) + g8 * 4 + t4;
                    const uint32_t* const xst = xlane + (size_t)c0 * 8;
                    if (nch == DEC_STAGE_CHUNKS) {
                        // a full stage: constant trip counts, no per-load conditions
#pragma unroll
                        for (int quad = 0; quad < DEC_STAGE_CHUNKS / (4 * DEC_WARPS); ++quad) {
                            uint32_t w[4][4], b[4][2];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int cc = warp + DEC_WARPS * (4 * quad + i);
#pragma unroll
                                for (int r = 0; r < 4; ++r) w[i][r] = wslot[cc * 128 + r * 32];
                                b[i][0] = xst[cc * 8];
                                b[i][1] = xst[cc * 8 + 4];
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (!col_live) { b[i][0] = 0u; b[i][1] = 0u; }
                                mma_s8(a[i][0], (w[i][0] << 4) & 0xF0F0F0F0u, (w[i][1] << 4) & 0xF0F0F0F0u, w[i][0] & 0xF0F0F0F0u,
                                       w[i][1] & 0xF0F0F0F0u, b[i][0], b[i][1]);
                                mma_s8(a[i][1], (w[i][2] << 4) & 0xF0F0F0F0u, (w[i][3] << 4) & 0xF0F0F0F0u, w[i][2] & 0xF0F0F0F0u,
                                       w[i][3] & 0xF0F0F0F0u, b[i][0], b[i][1]);
                            }
                        }
                    } else {
                        // the K tail: fewer chunks than a stage holds (the count is a multiple of four)
                        for (int cc = warp; cc < nch; cc += DEC_WARPS) {
                            uint32_t w[4];
#pragma unroll
                            for (int r = 0; r < 4; ++r) w[r] = wslot[cc * 128 + r * 32];
                            const uint32_t b0 = col_live ? xst[cc * 8] : 0u, b1 = col_live ? xst[cc * 8 + 4] : 0u;
                            mma_s8(a[0][0], (w[0] << 4) & 0xF0F0F0F0u, (w[1] << 4) & 0xF0F0F0F0u, w[0] & 0xF0F0F0F0u, w[1] & 0xF0F0F0F0u, b0, b1);
                            mma_s8(a[0][1], (w[2] << 4) & 0xF0F0F0F0u, (w[3] << 4) & 0xF0F0F0F0u, w[2] & 0xF0F0F0F0u, w[3] & 0xF0F0F0F0u, b0, b1);
                        }
                    }
                }
                release_stage();
            }
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    red[red_index(warp, rows, g * 32 + m * 16 + g8 + (e >> 1) * 8, 2 * t4 + (e & 1))] =
                        (a[0][m][e] + a[1][m][e]) + (a[2][m][e] + a[3][m][e]);
        }
        if (TRACE && trace && j == my_items - 1) trace[5] = (unsigned long long)(clock64() - c_start);
        // ---- sum the warps' partial sums, dequantise, store
        bar_sync_contraction();
        const float ca = sw_a, cb = sw_b;
        if (j + 1 < my_items) load_channel_scales(item + ncta);
        if (compute && !failed && tok_out < M) {
            int v = 0, u = 0;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) {
                v += red[red_index(w, rows, lane, tok_out)];
                if (swiglu) u += red[red_index(w, rows, 32 + lane, tok_out)];
            }
            v >>= 4;   // exact: the unpacked weights are 16 x code
            u >>= 4;
            const int n = item * GROUP + lane;
            if (swiglu) {
                const float y = __fmul_rn(silu_poly(dequant(v, sx, ca)), dequant(u, sx, cb));
                reinterpret_cast<float*>(p.out)[(size_t)tok_out * p.F + n] = y;
                run_max = max(run_max, __float_as_uint(y) & 0x7fffffffu);
            } else if (n < p.N) {
                if (p.epi == EPI_I32) reinterpret_cast<int*>(p.out)[(size_t)tok_out * p.N + n] = v;
                else if (p.epi == EPI_F32) reinterpret_cast<float*>(p.out)[(size_t)tok_out * p.N + n] = dequant(v, sx, ca);
                else reinterpret_cast<__half*>(p.out)[(size_t)tok_out * p.N + n] = __float2half_rn(dequant(v, sx, ca));
            }
        }
        if (j + 1 < my_items) bar_sync_contraction();   // the scratch is written again by the next item
    }
    if (TRACE && trace) trace[6] = (unsigned long long)(clock64() - c_start);
    if (swiglu && p.rowmax_out && compute) {
        const uint32_t m = __reduce_max_sync(0xffffffffu, run_max);   // a warp's 32 threads share one token
        if (lane == 0 && m && tok_out < M) atomicMax(&p.rowmax_out[tok_out], m);
    }

    // ---- bookkeeping
    if (failed && lane == 0) *reinterpret_cast<volatile int*>(&p.status->device_error) = 1;   // (a plain store: the block may be page-locked host memory)
    if (TRACE && trace) trace[7] = global_ns();
    if (tid == 0) {
        if (cta == 0) p.status->bad_input = verdict;
        if (no_scan) {
            // Every CTA has read the collected maxima by now; the last one to get here clears them
            // for the next SwiGLU epilogue.  The ticket counter wraps by itself.
            __threadfence();
            if (atomicInc(&p.status->done, nctas - 1u) == nctas - 1u)
                for (int t = 0; t < M; ++t) p.rowmax_in[t] = 0u;
        }
    }
}

template <bool HALF, bool TRACE>
__global__ void __launch_bounds__(DEC_THREADS, 2) gemm_decode_kernel(const DecodeParams p)
{
    decode_cta<HALF, TRACE>(p, blockIdx.x, gridDim.x);
}

// Several INDEPENDENT linears (same token count, activation type and cluster size) in one launch: the grid is the
// concatenation of their CTAs.  A decoder layer's q/k/v (or gate/up) projections read the same activations and
// do not depend on each other; launched one by one on a stream each would wait for the one in front, in one
// launch they pay the dependent latency once while their weights stream together.
template <bool HALF>
__global__ void __launch_bounds__(DEC_THREADS, 2) gemm_decode_batch_kernel(const DecodeBatch b)
{
    int i = 0;
    while (i + 1 < b.count && (int)blockIdx.x >= b.first_cta[i + 1]) ++i;
    decode_cta<HALF, false>(b.p[i], blockIdx.x - (unsigned)b.first_cta[i], (unsigned)(b.first_cta[i + 1] - b.first_cta[i]));
}

// ---------------------------------------------------------------------------------- host side
size_t gemm_decode_smem_bytes(int M, int KB, bool swiglu, int ring) { return dec_smem_bytes(M, KB, swiglu, ring); }

bool gemm_decode_supported(int M, int K)
{
    const int KB = (K + KBLOCK - 1) / KBLOCK;
    return M >= 1 && M <= 8 && (long long)KB * KBLOCK <= 131072 && dec_smem_bytes(M, KB, true, 2) <= DEC_SMEM_LIMIT;
}

// Ring depth: as deep as fits beside a second launch on the same SM (so that the next launch's CTAs, which
// request their weights before their dependency wait, are resident while this one runs); problems whose
// activation codes alone take most of that share get what one CTA per SM allows.
int gemm_decode_ring(int M, int KB, bool swiglu)
{
    const size_t fixed = dec_fixed_bytes(M, KB, swiglu) + 256;
    const size_t stage = DEC_STAGE_BYTES + 16, shared_budget = 112 * 1024;
    int ring = fixed < shared_budget ? (int)((shared_budget - fixed) / stage) : 0;
    if (ring < 2) {
        ring = fixed < DEC_SMEM_LIMIT ? (int)((DEC_SMEM_LIMIT - fixed) / stage) : 0;
        if (ring > 4) ring = 4;
    }
    return ring < DEC_MAX_RING ? ring : DEC_MAX_RING;
}

// Cluster size (= how many CTAs share the quantisation).  Quantising a 16-element unit costs a thread about 500
// cycles of issue slots and the exchange about as much as one and a half units, so up to three units per thread
// stay local; beyond that four CTAs share (clusters of eight leave half of this GPU's SMs without a CTA).
int gemm_decode_cluster(int M, int KB)
{
    const long long units = (long long)dec_token_slots(M) * KB * 8;
    return units <= 768 ? 1 : 4;
}

// CTAs: every resident CTA that has an item to work on (a multiple of the cluster size).  A launch lasts as long as
// its busiest CTA, ceil(items / CTAs) items, which no smaller grid improves; more CTAs bring more copy engines.
int gemm_decode_ctas(int items, int cluster, int cap)
{
    cap = cap / cluster * cluster;
    if (cap < cluster) cap = cluster;
    const int need = (items + cluster - 1) / cluster * cluster;
    return need <= cap ? need : cap;
}

template <bool HALF, bool TRACE>
static cudaError_t launch_decode_inst(const DecodeParams& p, cudaStream_t stream, bool pdl)
{
    auto kernel = gemm_decode_kernel<HALF, TRACE>;
    static PerDeviceOnce configured;
    int device = -1;
    if (configured.needed(device)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        configured.mark(device);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.ctas, 1, 1);
    cfg.blockDim = dim3(DEC_THREADS);
    cfg.dynamicSmemBytes = dec_smem_bytes(p.M, p.KB, p.epi == EPI_SWIGLU, p.ring);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (p.cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)p.cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
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

cudaError_t launch_gemm_decode(const DecodeParams& p, cudaStream_t stream, bool pdl)
{
    const bool swiglu = p.epi == EPI_SWIGLU;
    if (p.M < 1 || p.M > 8 || (p.cluster != 1 && p.cluster != 2 && p.cluster != 4 && p.cluster != 8) || p.ring < 2 ||
        p.ring > DEC_MAX_RING || p.ctas < p.cluster || p.ctas % p.cluster || (swiglu && p.F % GROUP) ||
        dec_smem_bytes(p.M, p.KB, swiglu, p.ring) > DEC_SMEM_LIMIT || (long long)p.KB * KBLOCK > 131072)
        return cudaErrorInvalidValue;
    if (p.trace) return p.half ? launch_decode_inst<true, true>(p, stream, pdl) : launch_decode_inst<false, true>(p, stream, pdl);
    return p.half ? launch_decode_inst<true, false>(p, stream, pdl) : launch_decode_inst<false, false>(p, stream, pdl);
}

template <bool HALF>
static cudaError_t launch_decode_batch_inst(const DecodeBatch& b, cudaStream_t stream, bool pdl)
{
    auto kernel = gemm_decode_batch_kernel<HALF>;
    static PerDeviceOnce configured;
    int device = -1;
    if (configured.needed(device)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        configured.mark(device);
    }
    size_t smem = 0;
    for (int i = 0; i < b.count; ++i) {
        const size_t need = dec_smem_bytes(b.p[i].M, b.p[i].KB, b.p[i].epi == EPI_SWIGLU, b.p[i].ring);
        smem = need > smem ? need : smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)b.first_cta[b.count], 1, 1);
    cfg.blockDim = dim3(DEC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (b.p[0].cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)b.p[0].cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, b);
}

// All linears of a batch: same M, activation type and cluster size; grid pieces are multiples of the cluster size.
cudaError_t launch_gemm_decode_batch(const DecodeBatch& b, cudaStream_t stream, bool pdl)
{
    if (b.count < 1 || b.count > DEC_MAX_BATCH || b.first_cta[0] != 0) return cudaErrorInvalidValue;
    for (int i = 0; i < b.count; ++i) {
        const DecodeParams& p = b.p[i];
        const bool swiglu = p.epi == EPI_SWIGLU;
        if (p.M != b.p[0].M || p.half != b.p[0].half || p.cluster != b.p[0].cluster || p.trace || p.M < 1 || p.M > 8 ||
            (p.cluster != 1 && p.cluster != 2 && p.cluster != 4 && p.cluster != 8) || p.ring < 2 || p.ring > DEC_MAX_RING ||
            p.ctas < p.cluster || p.ctas % p.cluster || b.first_cta[i + 1] - b.first_cta[i] != p.ctas || (swiglu && p.F % GROUP) ||
            dec_smem_bytes(p.M, p.KB, swiglu, p.ring) > DEC_SMEM_LIMIT || (long long)p.KB * KBLOCK > 131072)
            return cudaErrorInvalidValue;
    }
    return b.p[0].half ? launch_decode_batch_inst<true>(b, stream, pdl) : launch_decode_batch_inst<false>(b, stream, pdl);
}

// Resident clusters of this kernel with `smem` bytes of dynamic shared memory, times the cluster size:
// the most CTAs a launch may have if all of them are to run at once.
int gemm_decode_resident_ctas(int cluster, size_t smem, int sm_count)
{
    auto kernel = gemm_decode_kernel<true, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_LIMIT) != cudaSuccess) {
        cudaGetLastError();
        return sm_count / cluster * cluster;
    }
    if (cluster == 1) return sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster, 1, 1);
    cfg.blockDim = dim3(DEC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) {
        cudaGetLastError();
        return sm_count / cluster * cluster;
    }
    const int ctas = clusters * cluster;
    return ctas < sm_count ? ctas : sm_count / cluster * cluster;   // never more than one CTA per SM
}

} // namespace rkb200
