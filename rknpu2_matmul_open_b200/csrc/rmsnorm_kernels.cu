// rmsnorm_kernels.cu -- residual add + RMSNorm on fp16 tensors (rk_npu_add_rmsnorm_f16.h), one launch.
//
//   sum  = fp16(float(x) + float(residual))                                   -> residual_out
//   norm = fp16(float(double(sum) * inv * double(gamma))),  inv = 1 / sqrt(sum of double(sum)^2 / D + eps)   -> norm_out
//
// the double-precision statement of the original's board test (tests/test_add_rmsnorm_f16.cpp:96-113), which is what
// the original device's result is checked against.  Double-precision conversions run at a quarter of the fp32 rate and
// would be the busiest pipe of this kernel, so the second pass proves per value that single precision
// gives the same fp16 bits and falls back to the defining expression where it cannot (scale_one).
//
// HBM-bound: 4 tensors of 2 M D bytes cross DRAM once each.  A tile of TM tokens is shared by a CLUSTER of CS CTAs,
// each taking a slice of D: the sums stay in that CTA's shared memory between the two passes (both outputs are stored
// in the second one, so that no global store is in flight at the cluster barrier), the per-token sums of squares are exchanged through distributed shared memory and added in rank
// order by every CTA, so that the result does not depend on the schedule.  Both tensor layouts move 16-byte chunks
// (8 elements): in the block-8 layout (D/8, M, 8) consecutive TOKENS of one chunk column are contiguous, in row-major
// [M, D] consecutive CHUNKS of one token are; the thread index is split accordingly so that a warp touches 512
// contiguous bytes either way.
#include "rmsnorm_device.h"
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <atomic>
#include <cstdio>
#include <cstdlib>

namespace cg = cooperative_groups;

namespace rkb200 {
namespace {

constexpr int RN_THREADS = 512;
constexpr int RN_BATCH = 4;     // chunks of each input a thread requests before it uses the first
constexpr int RN_CTAS = 2;      // CTAs per SM the register allocation is bounded for
constexpr int RN_MAX_DEVICES = 64;
constexpr int RN_SMEM_SUMS = 64 * 1024;   // most bytes of sums one CTA keeps: TM * ceil(D/8/CS) * 16

__device__ __forceinline__ uint4 ld_stream(const uint4* p)
{
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(uint4* p, const uint4& v)
{
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// fp16(float(a) + float(b)) for a packed pair.  With 24 >= 2 * 11 + 2 mantissa bits the float sum rounded to fp16 equals
// the correctly rounded fp16 sum (double rounding is innocuous), which is what the packed fp16 add returns.  The squares
// of the two sums are added to acc in element order.
__device__ __forceinline__ uint32_t add_pair(uint32_t a, uint32_t b, double& acc)
{
    const __half2 s = __hadd2_rn(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    const float2 fs = __half22float2(s);
    const double lo = double(fs.x), hi = double(fs.y);
    acc += lo * lo;       // a product of two fp16 values is exact in double
    acc += hi * hi;
    return *reinterpret_cast<const uint32_t*>(&s);
}
// One output: fp16(float(double(v) * inv * double(g))), the defining expression, evaluated in double only when needed.
// y = fl32(fl32(v * inv_f) * g) with inv_f = fl32(inv) differs from the exact product x by at most 3 * 2^-24 |x|, and
// the float the defining expression rounds to fp16 by at most (2^-24 + 2^-52) |x|: the two are less than 4.000001
// float ulps apart.  fp16 rounding of a float in the normal fp16 range is decided by its low 13 mantissa bits L
// against the midpoint 0x1000; when |L - 0x1000| >= 8 no midpoint lies between the two floats (or on one of them), so
// fp16(y) IS the defined result.  About 0.2 % of the values, everything outside the normal fp16 range, and rows whose
// inv is not a normal float are not proven and are evaluated in double.

// The defining expression.  A real call, so that this rare path is branched around instead of being evaluated for
// every value (checking per value and not per chunk keeps the double-precision conversions, the slowest instructions
// here, to the values that need them).
__device__ __noinline__ float scale_defined(float v, float g, double inv) { return __double2float_rn(double(v) * inv * double(g)); }
__device__ __forceinline__ float scale_one(float v, float g, double inv, float inv_f, bool fast)
{
    float y = __fmul_rn(__fmul_rn(v, inv_f), g);
    const uint32_t u = __float_as_uint(y);
    const bool proven = fast && fabsf(y) >= 6.103515625e-05f && fabsf(y) < 65536.f      // 2^-14 <= |y| < 2^16 (false for NaN)
                        && ((u - (0x1000u - 7u)) & 0x1fffu) > 14u;                      // |L - 0x1000| >= 8
    if (!proven) y = scale_defined(v, g, inv);
    return y;
}
__device__ __forceinline__ uint32_t scale_pair(uint32_t v, uint32_t g, double inv, float inv_f, bool fast)
{
    const float2 fv = __half22float2(*reinterpret_cast<const __half2*>(&v));
    const float2 fg = __half22float2(*reinterpret_cast<const __half2*>(&g));
    const __half2 o = __floats2half2_rn(scale_one(fv.x, fg.x, inv, inv_f, fast), scale_one(fv.y, fg.y, inv, inv_f, fast));
    return *reinterpret_cast<const uint32_t*>(&o);
}

// ROWS: row-major [M, D]; else block-8 (D/8, M, 8).  grid = tiles * CS CTAs in clusters of CS.
template <bool ROWS>
__global__ void __launch_bounds__(RN_THREADS, RN_CTAS) add_rmsnorm_kernel(AddRmsNormParams p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int CS = int(cluster.num_blocks()), rank = int(cluster.block_rank());
    const int TM = p.tile_tokens, JL = RN_THREADS / TM;       // tokens of the tile x chunk lanes
    const int tid = threadIdx.x;
    const int dm = ROWS ? tid / JL : tid % TM, jl = ROWS ? tid % JL : tid / TM;
    const int m = int(blockIdx.x / CS) * TM + dm;
    const int chunks = p.D / 8, per = (chunks + CS - 1) / CS;
    const int j0 = min(chunks, rank * per), j1 = min(chunks, j0 + per);
    const bool live = m < p.M;

    uint4* s_sum = reinterpret_cast<uint4*>(smem);                               // this CTA's slice of the tile's sums
    double* s_part = reinterpret_cast<double*>(smem + size_t(TM) * per * 16);    // [RN_THREADS]
    double* s_token = s_part + RN_THREADS;                                       // [TM] this CTA's sum of squares per token
    auto lane_of = [&](int token, int lane) { return ROWS ? token * JL + lane : lane * TM + token; };
    auto global_at = [&](int j) { return ROWS ? size_t(m) * chunks + j : size_t(j) * p.M + m; };
    auto shared_at = [&](int j) { return ROWS ? dm * per + (j - j0) : (j - j0) * TM + dm; };

    double acc = 0.0;
    if (live) {
        for (int j = j0 + jl; j < j1; j += RN_BATCH * JL) {      // RN_BATCH chunks of both inputs in flight per thread
            uint4 a[RN_BATCH], b[RN_BATCH];
#pragma unroll
            for (int u = 0; u < RN_BATCH; ++u)
                if (j + u * JL < j1) {
                    const size_t at = global_at(j + u * JL);
                    a[u] = ld_stream(p.x + at);
                    b[u] = ld_stream(p.residual + at);
                }
#pragma unroll
            for (int u = 0; u < RN_BATCH; ++u)
                if (j + u * JL < j1) {
                    uint4 s;
                    s.x = add_pair(a[u].x, b[u].x, acc);
                    s.y = add_pair(a[u].y, b[u].y, acc);
                    s.z = add_pair(a[u].z, b[u].z, acc);
                    s.w = add_pair(a[u].w, b[u].w, acc);
                    s_sum[shared_at(j + u * JL)] = s;
                }
        }
    }
    s_part[tid] = acc;
    __syncthreads();
    if (JL <= 16) {                                            // few lanes per token: one thread adds them in lane order
        if (jl == 0) {
            double sum = acc;
            for (int lane = 1; lane < JL; ++lane) sum += s_part[lane_of(dm, lane)];
            s_token[dm] = sum;
        }
    } else {
        for (int step = JL / 2; step > 0; step >>= 1) {        // fixed tree over the chunk lanes of each token
            if (jl < step) s_part[tid] += s_part[lane_of(dm, jl + step)];
            __syncthreads();
        }
        if (jl == 0) s_token[dm] = s_part[tid];
    }
    if (CS > 1) cluster.sync(); else __syncthreads();
    double total = 0.0;
    for (int r = 0; r < CS; ++r) total += CS > 1 ? cluster.map_shared_rank(s_token, r)[dm] : s_token[dm];
    const double inv = 1.0 / sqrt(total / double(p.D) + double(p.eps));
    const float inv_f = __double2float_rn(inv);
    const bool fast = inv_f >= 1.17549435e-38f && inv_f <= 3.402823466e38f;       // a normal float (false for NaN)

    if (live) {
#pragma unroll 4
        for (int j = j0 + jl; j < j1; j += JL) {
            const uint4 s = s_sum[shared_at(j)];
            const uint4 g = __ldg(p.gamma + j);
            st_stream(p.residual_out + global_at(j), s);
            uint4 o;
            o.x = scale_pair(s.x, g.x, inv, inv_f, fast);
            o.y = scale_pair(s.y, g.y, inv, inv_f, fast);
            o.z = scale_pair(s.z, g.z, inv, inv_f, fast);
            o.w = scale_pair(s.w, g.w, inv, inv_f, fast);
            st_stream(p.norm_out + global_at(j), o);
        }
    }
    // A CTA's s_token must stay readable until every peer has read it.  Nothing this CTA wrote has to become visible
    // for that, so the arrival is relaxed: a releasing one would wait for the output stores still in flight.
    if (CS > 1) {
        asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    }
}

} // namespace

// Tile and cluster.  Candidates: tokens per tile a power of two up to 32 and up to the batch (in the block-8 layout
// at least 8 where the batch has them, so that a tile's chunks of one column are 128 contiguous bytes); clusters of
// 1, 2, 4 or 8 CTAs over D; the CTA's slice of the sums within RN_SMEM_SUMS; every thread of a cluster member with at
// least one chunk.  Taken: the candidate with the most CTAs up to 128 (small batches are spread over the GPU), then
// the smallest cluster, then the most tokens per tile.  Measured on 4096 rows: time falls with the work per CTA (a
// CTA's fixed cost -- start, load latency, two barriers, store drain -- is about 4 us) and rises with the cluster size.
void add_rmsnorm_geometry(int M, int D, int row_major, int& tile_tokens, int& cluster)
{
    int top = 1;
    while (top < 32 && top < M) top <<= 1;
    const int floor_tokens = row_major ? 1 : (top < 8 ? top : 8);
    const int chunks = D / 8;
    if (const char* text = std::getenv("RK_NPU_B200_RMSNORM_TILE")) {      // experiments: "tokens,cluster"
        int tm = 0, cs = 0;
        if (std::sscanf(text, "%d,%d", &tm, &cs) == 2 && tm >= 1 && tm <= 32 && (tm & (tm - 1)) == 0 && (cs == 1 || cs == 2 || cs == 4 || cs == 8) &&
            size_t(tm) * ((chunks + cs - 1) / cs) * 16 <= size_t(RN_SMEM_SUMS)) {
            tile_tokens = tm;
            cluster = cs;
            return;
        }
    }
    int best_score = -1;
    tile_tokens = 1;
    cluster = 8;        // D <= 32768: 512 chunks per CTA, one per thread
    for (int pass = 0; pass < 2 && best_score < 0; ++pass)      // second pass: without the block-8 floor, if nothing fitted
        for (int cs = 1; cs <= 8; cs <<= 1)
            for (int tm = top; tm >= (pass ? 1 : floor_tokens); tm >>= 1) {
                const int per = (chunks + cs - 1) / cs;
                if (size_t(tm) * per * 16 > size_t(RN_SMEM_SUMS)) continue;
                if (cs > 1 && tm * per < RN_THREADS) continue;
                const int ctas = (M + tm - 1) / tm * cs;
                const int score = ctas < 128 ? ctas : 128;
                if (score > best_score) {
                    best_score = score;
                    tile_tokens = tm;
                    cluster = cs;
                }
            }
}

cudaError_t launch_add_rmsnorm(const AddRmsNormParams& q, cudaStream_t stream)
{
    AddRmsNormParams p = q;
    int cs = 1;
    add_rmsnorm_geometry(p.M, p.D, p.row_major, p.tile_tokens, cs);
    const int per = (p.D / 8 + cs - 1) / cs;
    const size_t shared = size_t(p.tile_tokens) * per * 16 + size_t(RN_THREADS + p.tile_tokens) * sizeof(double);
    auto kernel = p.row_major ? add_rmsnorm_kernel<true> : add_rmsnorm_kernel<false>;
    // function attributes are per device: remember what this device's copy of the kernel already allows
    static std::atomic<int> allowed[2][RN_MAX_DEVICES];
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    std::atomic<int>* known = device >= 0 && device < RN_MAX_DEVICES ? &allowed[p.row_major ? 1 : 0][device] : nullptr;
    if (!known || known->load(std::memory_order_relaxed) < int(shared)) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(RN_SMEM_SUMS + (RN_THREADS + 32) * sizeof(double)));
        if (err != cudaSuccess) return err;
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, int(cudaSharedmemCarveoutMaxShared));
        if (err != cudaSuccess) return err;
        if (known) known->store(int(RN_SMEM_SUMS + (RN_THREADS + 32) * sizeof(double)), std::memory_order_relaxed);
    }
    cudaLaunchConfig_t cfg{};
    const int tiles = (p.M + p.tile_tokens - 1) / p.tile_tokens;
    cfg.gridDim = dim3(unsigned(tiles) * unsigned(cs));
    cfg.blockDim = dim3(RN_THREADS);
    cfg.dynamicSmemBytes = shared;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = unsigned(cs);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

} // namespace rkb200
