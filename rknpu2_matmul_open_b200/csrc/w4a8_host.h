// w4a8_host.h -- host-side objects behind the opaque handles of the C ABI.
#pragma once
#include "../../include/rknpu_b200_ext.h"
#include "w4a8_device.h"
#include <atomic>
#include <cuda_runtime.h>
#include <mutex>
#include <string>

struct rk_npu_ctx {
    int device = 0;
    uint64_t id = 0;              // cookie compared by the DOMAIN checks
    uint32_t driver_version = 0;  // CUDA driver version; part of the tuning-cache key
    int sm_count = 0;
    cudaStream_t stream = nullptr;  // weight uploads
    // group of GPUs (rk_npu_b200_open_group): this context is `rank` of `world`; comm is the NCCL communicator
    int rank = 0, world = 1;
    void* comm = nullptr;
};

struct rk_npu_iommu_domain {
    rk_npu_ctx* ctx = nullptr;
    uint32_t id = 0;
    std::atomic<int> refs{1};
    std::mutex lock;
    rk_npu_domain_memory_stats stats{};
};

namespace rkb200 {

// Weight identity and certified K tiles captured at creation
// (the reference's w4_tune::Profile, src/rk_npu_w4a8_tune_internal.h:27-34).
struct Profile {
    int K = 0, N = 0, safe = 0, limit = 0;
    double multiplier = 1;
    uint64_t fingerprint = 0, safe_tiles = 0;
    bool certified(int k) const { return k >= 32 && k <= 2048 && k % 32 == 0 && (safe_tiles & (uint64_t(1) << (k / 32 - 1))); }
    bool permits(int k) const { return k >= 32 && k <= limit && k % 32 == 0 && (certified(k) || multiplier > 1); }
    rk_npu_w4a8_weight_info info(int k) const { return {{K, N, k}, safe, multiplier, !certified(k)}; }
};

struct WeightBound {
    int k_tile = 0;
    int64_t positive = 0, negative_magnitude = 0;
    uint64_t safe_tiles = 0;
};
int bound_weights(int K, int N, const int8_t* B, int requested, WeightBound& out, int fallback = 0);
uint64_t weight_fingerprint(int K, int N, const int8_t* B, const float* scales);
int make_profile(const rk_npu_w4a8_autotune_config& c, const int8_t* B, const float* scale, Profile& out);
bool valid_autotune_config(const rk_npu_w4a8_autotune_config& c);
rk_npu_w4a8_weights* create_weights(rk_npu_iommu_domain* domain, const rk_npu_w4a8_weight_info& info, const int8_t* B,
                                    const float* scales, const Profile* profile);
const Profile& weights_profile(const rk_npu_w4a8_weights* w);

void domain_retain(rk_npu_iommu_domain* d);
void domain_release(rk_npu_iommu_domain* d);
// Device allocations are accounted to the owning domain.
int device_alloc(rk_npu_iommu_domain* d, void** ptr, size_t bytes);
void device_free(rk_npu_iommu_domain* d, void* ptr, size_t bytes);

// ---- group of GPUs (w4a8_group.cpp)
void group_close(rk_npu_ctx* ctx);
int group_all_gather(rk_npu_ctx* ctx, void* buffer, size_t bytes_per_rank, cudaStream_t stream);
int group_all_reduce_max_u32(rk_npu_ctx* ctx, uint32_t* values, size_t count, cudaStream_t stream);
// Columns of a weight [K, N] this rank holds: N % 128 == 0 -> the same slice [f0, f1) of both halves of N
// (so that a [gate | up] packing keeps its SwiGLU pairs on one GPU; `two_range`), else one contiguous run.
struct ShardPlan {
    bool two_range = false;
    int n0 = 0, n1 = 0;          // slice of N (contiguous) or of N / 2 (two_range)
    int columns() const { return (two_range ? 2 : 1) * (n1 - n0); }
};
inline ShardPlan shard_plan(int N, int world, int rank)
{
    ShardPlan p;
    p.two_range = world > 1 && N % 128 == 0;
    shard_range(p.two_range ? N / 2 : N, world, rank, p.n0, p.n1);
    return p;
}

inline int align_up(int x, int a) { return (x + a - 1) / a * a; }
inline int64_t align_up64(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

} // namespace rkb200

struct rk_npu_w4a8_weights {
    rk_npu_iommu_domain* domain = nullptr;
    uint64_t ctx_id = 0;
    uint32_t domain_id = 0;
    rk_npu_w4a8_weight_info info{};
    rkb200::Profile profile;
    uint8_t* packed = nullptr;  // Wp
    float* scales = nullptr;    // padded to 32*NG
    size_t packed_bytes = 0, scale_bytes = 0;
    int KB = 0, NG = 0;
    rkb200::ShardPlan shard;    // the columns this object holds (all of them outside a group)
    int shard_N = 0;            // == shard.columns()
};

struct rk_npu_w4a8_workspace {
    rk_npu_w4a8_config config{};
    rk_npu_iommu_domain* domain = nullptr;
    uint64_t ctx_id = 0;
    uint32_t domain_id = 0;
    bool npu_reduce = false;
    int input_layout = 0;
    std::atomic_flag busy = ATOMIC_FLAG_INIT;
    cudaStream_t stream = nullptr;
    // geometry
    bool pair = false; // tcgen05 path runs two-CTA tiles
    int T = 0;        // token tile of the code layout
    int TC = 0;       // tokens per CTA of the mma.sync kernel (0 when the tcgen05 kernel is used)
    int KB = 0;       // k-blocks
    int tiles_per_cta_override = 0;        // single-kernel path: 0 = automatic, 1 or 2 (RK_NPU_B200_TILES_PER_CTA)
    int variant = 0, split_override = 0;   // variant: 1 quantise + mma.sync GEMM, 2 quantise + tcgen05 GEMM, 3 fused small batch
                                           // (split-K clusters), 4 quantise + persistent streaming GEMM (small batch, large
                                           // weights), 5 single-kernel decode (whole-K CTAs, up to eight tokens)
    int decode_cap[4] = {0, 0, 0, 0};      // variant 5: CTAs resident at once for cluster sizes 1, 2, 4, 8
    bool starve = false;                   // test hook (rk_npu_b200_w4a8_test_starve): first weight barrier never completes
    // device buffers
    uint8_t* codes = nullptr;
    float* scales = nullptr;
    float* inverse = nullptr;
    uint32_t* rowmax = nullptr;
    int* partials = nullptr;          // variant 4: per-tile partial sums and k-block counters
    unsigned int* counts = nullptr;
    size_t partials_bytes = 0, counts_bytes = 0;
    rkb200::Status* status = nullptr;
    void* stage_in = nullptr;   // device copy of host activations
    void* stage_out = nullptr;  // device copy of host outputs
    size_t codes_bytes = 0, stage_in_bytes = 0, stage_out_bytes = 0;
    rkb200::Status* host_status = nullptr;  // pinned
    rkb200::Status* host_status_alias = nullptr;   // its device address (NULL if the GPU cannot address it)
    void* bounce_in = nullptr;        // page-locked pieces the blocking calls copy small ordinary host tensors through
    void* bounce_out = nullptr, *bounce_out_alias = nullptr;
    size_t bounce_bytes = 0;
    cudaEvent_t events[8]{};
    std::atomic<uint64_t> launches{0};
    unsigned long long* trace = nullptr;   // device stamps, allocated by rk_npu_b200_w4a8_trace_enable
    size_t trace_bytes = 0;
    // group of GPUs: the kernels compute `shard_N` columns into this rank's slot of `gather` (world slots of
    // gather_slot bytes: a compact [M][widest shard] block of 4-byte elements), an all-gather fills the others
    // and the rows are reassembled into the caller's tensor (or `stage_out` for a host caller)
    rkb200::ShardPlan shard;
    int shard_N = 0;
    uint8_t* gather = nullptr;
    size_t gather_slot = 0, gather_bytes = 0;
    uint8_t* code_gather = nullptr;     // all-gathered int8 activation codes of a group FFN's down projection
    size_t code_gather_bytes = 0;
};
