/*
 * rknpu_b200_w4a8.h -- C ABI of the B200 (sm_100a) W4A8 quantized-linear library.
 *
 * The library is a binary drop-in for the W4A8 path of rknpu2_matmul_open: every
 * type below has the layout, and every function the name, argument meaning and
 * error behaviour, of the interface it replaces.  A program built against the
 * original rk_npu_common.h / rk_npu_matmul_i4.h / rk_npu_w4a8.h / rk_npu_w4a8_tune.h
 * links against this library unchanged; this header exists so the library can be
 * built and used where those headers are not installed.  Each declaration names
 * the original declaration it stands for (file:line in the original project).
 *
 * What differs behind the ABI:
 *   - rk_npu_open(dev) opens one CUDA device: NULL or "" selects the device named
 *     by the RK_NPU_CUDA_DEVICE environment variable (default: the calling
 *     thread's current CUDA device), "cuda:N" selects device N.
 *   - Tensor arguments (A, C, middle) may be host pointers, as in the original,
 *     or device pointers on the context's GPU; device pointers skip all copies.
 *   - m_tile / n_tile / npu_core_mask / pipeline / cpu_threads / input layout /
 *     reduce backend are validated exactly as the original validates them and are
 *     then scheduling hints only; every choice produces the same numbers.
 *   - Integer accumulation is a direct int32 sum on the GPU, so an "uncertified"
 *     k_tile (multiplier > 1) cannot saturate here.
 *
 * Valid C99 and C++.
 */
#ifndef RKNPU_B200_W4A8_H
#define RKNPU_B200_W4A8_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status codes
 * include/rk_npu_common.h:28-37 */
#define RK_NPU_OK 0
#define RK_NPU_ERR_OPEN (-1)       /* no usable CUDA device / device could not be opened */
#define RK_NPU_ERR_IOCTL (-2)      /* a CUDA runtime call failed outside a kernel launch */
#define RK_NPU_ERR_PARAM (-3)      /* bad argument, non-finite activation, non-finite middle */
#define RK_NPU_ERR_NOMEM (-4)      /* an allocation failed or a size does not fit */
#define RK_NPU_ERR_SUBMIT (-5)     /* a kernel failed, or a bounded device wait ran out */
#define RK_NPU_ERR_BUSY (-6)       /* the workspace is running another call */
#define RK_NPU_ERR_DOMAIN (-7)     /* objects come from different contexts or domains */
#define RK_NPU_ERR_IO (-8)         /* file I/O failed */
#define RK_NPU_ERR_CACHE_MISS (-9) /* tuning cache absent, stale or malformed */

#define RK_NPU_IOMMU_DOMAIN_COUNT 16u /* include/rk_npu_common.h:61 */

/* ------------------------------------------------------------------ context, domains
 * include/rk_npu_common.h:75-76,126-127,132-135,157.  A domain is a logical pool tag
 * inside one context; objects made from different (context, domain) pairs refuse to
 * work together with RK_NPU_ERR_DOMAIN, as on the original device. */
typedef struct rk_npu_ctx rk_npu_ctx;
typedef struct rk_npu_iommu_domain rk_npu_iommu_domain;

rk_npu_ctx *rk_npu_open(const char *dev);
void rk_npu_close(rk_npu_ctx *ctx);
rk_npu_iommu_domain *rk_npu_iommu_domain_create(rk_npu_ctx *ctx, uint32_t domain_id);
void rk_npu_iommu_domain_free(rk_npu_iommu_domain *domain);
uint32_t rk_npu_iommu_domain_id(const rk_npu_iommu_domain *domain);
const char *rk_npu_strerror(int code);

/* include/rk_npu_common.h:141-145: device bytes owned through this domain. */
typedef struct {
    uint64_t live_bytes, peak_bytes, creates, destroys;
} rk_npu_domain_memory_stats;
int rk_npu_iommu_domain_memory_stats(const rk_npu_iommu_domain *domain, rk_npu_domain_memory_stats *stats);

/* ------------------------------------------------------------------ caller-owned device-visible buffers
 * include/rk_npu_common.h:39-46,63-73,94-106,160-190.  Here a buffer is page-locked host memory mapped into the GPU's
 * address space: vaddr is the host mapping, dma_addr (= obj_addr) the address kernels use; it is coherent once the call
 * that used it has returned, so rk_npu_mem_sync validates its arguments and does nothing else.  The allocation flags are
 * accepted and, except CACHEABLE (recorded in flags), without effect.  The dmabuf import and export are declined
 * (RK_NPU_ERR_PARAM): there is no dmabuf on this platform. */
#define RK_NPU_MEM_NON_CONTIGUOUS 0x1
#define RK_NPU_MEM_NON_CACHEABLE 0x0
#define RK_NPU_MEM_CACHEABLE 0x2
#define RK_NPU_MEM_WRITE_COMBINE 0x4
#define RK_NPU_MEM_KERNEL_MAPPING 0x8
#define RK_NPU_MEM_IOMMU 0x10
#define RK_NPU_MEM_IOMMU_LIMIT_IOVA_ALIGNMENT 0x400
#define RK_NPU_MEM_DATA_DEFAULT (RK_NPU_MEM_NON_CONTIGUOUS | RK_NPU_MEM_CACHEABLE | RK_NPU_MEM_IOMMU)
#define RK_NPU_MEM_DEFAULT RK_NPU_MEM_DATA_DEFAULT
#define RK_NPU_MEM_F_OWN_RKNPU (1u << 0) /* owns its storage */
#define RK_NPU_MEM_F_IMPORTED (1u << 1)
#define RK_NPU_MEM_F_VIEW (1u << 2)      /* non-owning subrange */
#define RK_NPU_MEM_F_MAPPED (1u << 3)    /* vaddr is valid */
#define RK_NPU_MEM_F_CACHEABLE (1u << 4)

typedef enum {
    RK_NPU_SYNC_TO_DEVICE = 1u << 0,
    RK_NPU_SYNC_FROM_DEVICE = 1u << 1,
} rk_npu_sync_dir;

typedef struct {
    uint32_t handle;   /* nonzero for a live base allocation */
    uint32_t flags;    /* RK_NPU_MEM_F_* */
    uint64_t obj_addr;
    uint64_t dma_addr; /* device address of this view */
    void *vaddr;       /* host address of this view */
    uint64_t size;     /* bytes of this view */
    uint64_t offset;   /* from the base allocation */
    uint64_t capacity; /* bytes of the base allocation */
    uint64_t ctx_id;
    uint32_t iommu_domain_id;
    uint32_t reserved;
} rk_npu_mem;

/* RK_NPU_ERR_PARAM: NULL domain / out, size 0; RK_NPU_ERR_NOMEM: the allocation failed. */
int rk_npu_mem_alloc(rk_npu_iommu_domain *domain, uint64_t size, uint32_t alloc_flags, rk_npu_mem *out);
int rk_npu_mem_view(const rk_npu_mem *base, uint64_t offset, uint64_t size, rk_npu_mem *out_view);
int rk_npu_mem_sync(rk_npu_ctx *ctx, const rk_npu_mem *mem, rk_npu_sync_dir dir);
/* Releases a base allocation, or clears a view; the struct is zeroed. */
int rk_npu_mem_free(rk_npu_ctx *ctx, rk_npu_mem *mem);
int rk_npu_mem_import_dmabuf(rk_npu_iommu_domain *domain, int dmabuf_fd, void *cpu_addr, uint64_t size,
                             uint32_t import_flags, rk_npu_mem *out);
int rk_npu_mem_export_dmabuf(rk_npu_ctx *ctx, const rk_npu_mem *mem, int *out_fd);

/* ------------------------------------------------------------------ int4 weight key
 * include/rk_npu_matmul_i4.h:22-25,38-46,58. */
typedef struct rk_npu_i4_weight_config {
    int K, N;
    int k_tile; /* multiple of 32 in 32..2048; above 480 the weights must certify it */
} rk_npu_i4_weight_config;

typedef struct rk_npu_i4_memory_info {
    uint64_t packed_weight_bytes;
    uint64_t input_bytes;
    uint64_t partial_bytes;
    uint64_t control_bytes;
    uint32_t wave_count;
    uint32_t tasks_per_wave;
} rk_npu_i4_memory_info;

int rk_npu_i4_weights_memory_query(const rk_npu_i4_weight_config *cfg, uint64_t *bytes);

/* ------------------------------------------------------------------ W4A8 configuration
 * include/rk_npu_w4a8.h:16-33 */
typedef enum rk_npu_w4a8_pipeline {
    RK_NPU_W4A8_SERIAL = 0,
    RK_NPU_W4A8_PIPELINED = 1,
    RK_NPU_W4A8_CHAIN = 2
} rk_npu_w4a8_pipeline;

typedef struct rk_npu_w4a8_config {
    int M, N, K;            /* tokens, output channels, reduction; K <= INT32_MAX/1024 */
    int m_tile;             /* 1..64 (1..256 with the panel8 option) */
    int k_tile;             /* 32..2048, multiple of 32; must equal the weights' k_tile */
    int n_tile;             /* 64..8128, multiple of 64 */
    uint32_t npu_core_mask; /* one of 1, 2, 4, 3, 7 */
    uint32_t timeout_ms;    /* > 0; bounds every device-side wait of a call */
    int pipeline;           /* rk_npu_w4a8_pipeline */
    int cpu_threads;        /* 1..4 */
} rk_npu_w4a8_config;

/* include/rk_npu_w4a8.h:35-40 */
typedef struct rk_npu_w4a8_memory_info {
    rk_npu_i4_memory_info backend;
    uint64_t weight_metadata_bytes;
    uint64_t cpu_scratch_bytes;
} rk_npu_w4a8_memory_info;

/* include/rk_npu_w4a8.h:51-63 */
typedef enum rk_npu_w4a8_input_layout {
    RK_NPU_W4A8_INPUT_NATIVE = 0,
    RK_NPU_W4A8_INPUT_PANEL8 = 1
} rk_npu_w4a8_input_layout;
typedef enum rk_npu_w4a8_reduce_backend {
    RK_NPU_W4A8_REDUCE_CPU = 0,
    RK_NPU_W4A8_REDUCE_NPU = 1
} rk_npu_w4a8_reduce_backend;
typedef struct rk_npu_w4a8_options {
    uint32_t struct_size; /* set by rk_npu_w4a8_options_init */
    rk_npu_w4a8_input_layout input_layout;
    rk_npu_w4a8_reduce_backend reduce_backend;
} rk_npu_w4a8_options;

/* include/rk_npu_w4a8.h:64-75 */
typedef struct rk_npu_w4a8_memory_info_ex {
    rk_npu_w4a8_memory_info base;
    uint64_t reduction_output_bytes;
    uint64_t reduction_weight_bytes;
    uint64_t reduction_control_bytes;
    uint64_t workspace_bytes;
    rk_npu_w4a8_reduce_backend effective_reduce_backend;
} rk_npu_w4a8_memory_info_ex;

/* include/rk_npu_w4a8.h:76-83.  On this library (device times from CUDA events, host times from the wall clock):
 *   activation_scan_us  the absmax + quantise kernel in front of a two-kernel GEMM (0 for the single-launch decode
 *                       kernel, which scans inside the GEMM launch, and for an FFN's down projection, which never scans)
 *   quant_pack_us       the re-quantise kernel of an FFN's down projection (scales from the collected row maxima)
 *   submit_us           the GEMM kernel(s); split-K reduction and dequantisation are fused into it, so dequant_us is 0
 *   reduce_us           in a group of GPUs: the all-gather and reassembly of the column shards; 0 on one GPU
 *   sync_us             host<->device copies plus the final stream wait
 *   total_us            the wall time of the blocking call */
typedef struct rk_npu_w4a8_timings {
    double activation_scan_us;
    double quant_pack_us, sync_us, submit_us, reduce_us;
    double dequant_us, total_us;
} rk_npu_w4a8_timings;

typedef struct rk_npu_w4a8_weights rk_npu_w4a8_weights;     /* include/rk_npu_w4a8.h:84 */
typedef struct rk_npu_w4a8_workspace rk_npu_w4a8_workspace; /* include/rk_npu_w4a8.h:85 */

/* include/rk_npu_w4a8.h:87-92 */
typedef struct rk_npu_w4a8_weight_info {
    rk_npu_i4_weight_config config;
    int safe_k_tile;
    double multiplier;
    int bound_relaxed;
} rk_npu_w4a8_weight_info;

/* include/rk_npu_w4a8.h:94-99 */
void rk_npu_w4a8_config_init(rk_npu_w4a8_config *cfg, int M, int N, int K);
int rk_npu_w4a8_memory_query(const rk_npu_w4a8_config *cfg, rk_npu_w4a8_memory_info *out);
void rk_npu_w4a8_options_init(rk_npu_w4a8_options *options);
int rk_npu_w4a8_memory_query_ex(const rk_npu_w4a8_config *cfg, const rk_npu_w4a8_options *options,
                                rk_npu_w4a8_memory_info_ex *out);

/* include/rk_npu_w4a8.h:114-127.  B[K,N] holds one int8 per int4 code in [-8,7];
 * w_scale[N] finite and > 0.  Both are copied (B is repacked on the GPU into the
 * streaming layout); the caller may free them.  k_tile == 0 picks the largest tile the
 * weights certify, scaled by RK_NPU_W4A8_K_TILE_MULTIPLIER.  NULL on any invalid input. */
rk_npu_w4a8_weights *rk_npu_w4a8_weights_create(rk_npu_iommu_domain *domain, const rk_npu_i4_weight_config *cfg,
                                                const int8_t *B, const float *w_scale);
void rk_npu_w4a8_weights_free(rk_npu_w4a8_weights *weights);
int rk_npu_w4a8_weights_query(const rk_npu_w4a8_weights *weights, rk_npu_w4a8_weight_info *info);
rk_npu_w4a8_workspace *rk_npu_w4a8_workspace_create(rk_npu_iommu_domain *domain, const rk_npu_w4a8_config *cfg);
rk_npu_w4a8_workspace *rk_npu_w4a8_workspace_create_ex(rk_npu_iommu_domain *domain, const rk_npu_w4a8_config *cfg,
                                                       const rk_npu_w4a8_options *options);
void rk_npu_w4a8_workspace_free(rk_npu_w4a8_workspace *workspace);

/* include/rk_npu_w4a8.h:144-147.  Blocking; A[M,K], C[M,N] compact row-major and
 * non-aliasing; fp16 travels as binary16 bit patterns.
 *   s[m] = max(max|A[m,:]| / 127, FLT_MIN)  (1 for an all-zero row)
 *   q    = clamp(round_half_away(A * (1/s)), -127, 127)
 *   C    = (float(sum_k q*B) * s[m]) * w_scale[n], rounded once more for fp16.
 * NaN/Inf in A -> RK_NPU_ERR_PARAM, no GEMM work done. */
int rk_npu_w4a8_run_f32(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights, const float *A,
                        float *C, rk_npu_w4a8_timings *timings);
int rk_npu_w4a8_run_f16(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights, const uint16_t *A,
                        uint16_t *C, rk_npu_w4a8_timings *timings);

/* include/rk_npu_w4a8.h:163-165.  N = 2F with weight columns [gate(F), up(F)];
 * middle[M,F] = (g / (1 + exp(-g))) * u.  Needs N % 64 == 0 and the CPU reduce option.
 * exp is the original's degree-7 polynomial (every rounding step reproduced). */
int rk_npu_w4a8_run_swiglu_f32(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights,
                               const float *A, float *middle, rk_npu_w4a8_timings *timings);

/* include/rk_npu_w4a8.h:167-170 */
typedef struct rk_npu_w4a8_ffn_timings {
    rk_npu_w4a8_timings gate_up, down;
    double total_us;
} rk_npu_w4a8_ffn_timings;

/* include/rk_npu_w4a8.h:186-189.  gate/up -> SwiGLU -> down.  The SwiGLU epilogue
 * collects each row's max |middle|; down quantises middle with the scale derived from
 * it without rescanning.  Non-finite middle -> RK_NPU_ERR_PARAM before down runs. */
int rk_npu_w4a8_run_ffn_f32(rk_npu_w4a8_workspace *gate_up, const rk_npu_w4a8_weights *gate_up_weights,
                            rk_npu_w4a8_workspace *down, const rk_npu_w4a8_weights *down_weights, const float *A,
                            float *middle, float *C, rk_npu_w4a8_ffn_timings *timings);

/* ------------------------------------------------------------------ tuning cache (load side)
 * include/rk_npu_w4a8_tune.h:8-44 */
typedef enum rk_npu_w4a8_activation_type { RK_NPU_W4A8_F32 = 0, RK_NPU_W4A8_F16 = 1 } rk_npu_w4a8_activation_type;

typedef struct rk_npu_w4a8_autotune_config {
    int M, N, K;
    rk_npu_w4a8_activation_type activation_type;
    uint32_t allowed_npu_core_mask;
    uint64_t allowed_cpu_core_mask;
    int warmup, loops, repeats;
    uint32_t timeout_ms;
    int verbose;
    int required_k_tile;
    double k_tile_multiplier;
} rk_npu_w4a8_autotune_config;

typedef struct rk_npu_w4a8_strategy {
    rk_npu_w4a8_config config;
    rk_npu_w4a8_activation_type activation_type;
    uint64_t cpu_core_mask;
    rk_npu_w4a8_weight_info weights;
    uint64_t weight_fingerprint;
    uint32_t tuning_revision;
    double input_us, npu_us, sync_us, output_us, total_us;
    double jitter_pct, robust_us;
} rk_npu_w4a8_strategy;

typedef struct rk_npu_w4a8_strategy_ex {
    rk_npu_w4a8_strategy base;
    rk_npu_w4a8_options execution;
} rk_npu_w4a8_strategy_ex;

/* include/rk_npu_w4a8_tune.h:50-60: weight identity and certified tiles captured at
 * weight creation; owns no device memory and may outlive the weights. */
typedef struct rk_npu_w4a8_tuning_profile rk_npu_w4a8_tuning_profile;
rk_npu_w4a8_tuning_profile *rk_npu_w4a8_tuning_profile_from_weights(const rk_npu_w4a8_weights *weights);
void rk_npu_w4a8_tuning_profile_free(rk_npu_w4a8_tuning_profile *profile);
uint64_t rk_npu_w4a8_tuning_profile_fingerprint(const rk_npu_w4a8_tuning_profile *profile);

/* include/rk_npu_w4a8_tune.h:80 */
void rk_npu_w4a8_autotune_config_init(rk_npu_w4a8_autotune_config *cfg, int M, int N, int K);

/* include/rk_npu_w4a8_tune.h:57-60: load-only lookup; no device work, no weight scan. */
int rk_npu_w4a8_autotune_cache_load_profile_ex(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg,
                                               const rk_npu_w4a8_tuning_profile *profile, const char *cache_path,
                                               rk_npu_w4a8_strategy_ex *fastest, rk_npu_w4a8_strategy_ex *stable);
/* include/rk_npu_w4a8_tune.h:112-117,147-152: lookups / writes that rescan the weights. */
int rk_npu_w4a8_autotune_cache_load(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg, const int8_t *B,
                                    const float *w_scale, const char *cache_path, rk_npu_w4a8_strategy *fastest,
                                    rk_npu_w4a8_strategy *stable);
int rk_npu_w4a8_autotune_cache_save(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg, const int8_t *B,
                                    const float *w_scale, const char *cache_path,
                                    const rk_npu_w4a8_strategy *fastest, const rk_npu_w4a8_strategy *stable);
int rk_npu_w4a8_autotune_cache_load_ex(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg, const int8_t *B,
                                       const float *w_scale, const char *cache_path,
                                       rk_npu_w4a8_strategy_ex *fastest, rk_npu_w4a8_strategy_ex *stable);
int rk_npu_w4a8_autotune_cache_save_ex(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg, const int8_t *B,
                                       const float *w_scale, const char *cache_path,
                                       const rk_npu_w4a8_strategy_ex *fastest,
                                       const rk_npu_w4a8_strategy_ex *stable);

/* include/rk_npu_w4a8_tune.h:122-123,153-158: factories driven by a (loaded) strategy. */
rk_npu_w4a8_weights *rk_npu_w4a8_weights_create_tuned(rk_npu_iommu_domain *domain,
                                                      const rk_npu_w4a8_strategy *strategy, const int8_t *B,
                                                      const float *w_scale);
rk_npu_w4a8_weights *rk_npu_w4a8_weights_create_tuned_ex(rk_npu_iommu_domain *domain,
                                                         const rk_npu_w4a8_strategy_ex *strategy, const int8_t *B,
                                                         const float *w_scale);
rk_npu_w4a8_workspace *rk_npu_w4a8_workspace_create_tuned_ex(rk_npu_iommu_domain *domain,
                                                             const rk_npu_w4a8_strategy_ex *strategy);

/* ------------------------------------------------------------------ search tuner
 * include/rk_npu_w4a8_tune.h:62-167.  The original searches tiles, host teams and pipeline modes of
 * its three-core device.  On this library the search space is: which kernel family runs the shape
 * (single-launch decode kernel, mma.sync split-K ring, tcgen05 per-tile / persistent / streaming
 * kernels) and how many CTAs cooperate on a column tile (split-K factor / cluster size).  The
 * protocol is the original's: complete blocking calls on a deterministic calibration tensor, the
 * first result checked against the int64 formula, every later output compared with it, warm-up,
 * loops x repeats, median, jitter and robust figures.  Candidates are ranked by the device part of
 * the call (host copies are the same for all of them); total_us / robust_us record the whole call.
 * The winner is written into the strategy's existing fields -- pipeline, m_tile, n_tile keep their
 * names, ranges and validity rules and select the schedule (rk_npu_w4a8_workspace_create_tuned_ex
 * honours them; rk_npu_w4a8_workspace_create[_ex] keeps choosing by itself):
 *   pipeline  CHAIN: single-launch decode kernel; SERIAL: quantise + mma.sync ring; PIPELINED: see m_tile
 *   m_tile    64 automatic; 32 mma.sync ring; 48 tcgen05 streaming kernel; 56 tcgen05 tile kernel
 *   n_tile    128 / 256 / 512 / 1024: 1 / 2 / 4 / 8 cooperating CTAs; anything else automatic
 * Either output may be NULL, not both.  Needs a context opened on a GPU. */
int rk_npu_w4a8_autotune(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg, const int8_t *B, const float *w_scale,
                         rk_npu_w4a8_strategy *fastest, rk_npu_w4a8_strategy *stable);
int rk_npu_w4a8_autotune_ex(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg, const int8_t *B,
                            const float *w_scale, rk_npu_w4a8_strategy_ex *fastest, rk_npu_w4a8_strategy_ex *stable);
/* A valid cache file answers without device work (cache_hit = 1) unless refresh; otherwise search and save
 * (a failed save leaves the strategies valid).  NULL cache_path: the default location. */
int rk_npu_w4a8_autotune_cached(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg, const int8_t *B,
                                const float *w_scale, const char *cache_path, int refresh, rk_npu_w4a8_strategy *fastest,
                                rk_npu_w4a8_strategy *stable, int *cache_hit);
int rk_npu_w4a8_autotune_cached_ex(rk_npu_ctx *ctx, const rk_npu_w4a8_autotune_config *cfg, const int8_t *B,
                                   const float *w_scale, const char *cache_path, int refresh,
                                   rk_npu_w4a8_strategy_ex *fastest, rk_npu_w4a8_strategy_ex *stable, int *cache_hit);

/* include/rk_npu_w4a8_tune.h:62-73: several batch sizes of one weight, sharing one K partition. */
typedef struct rk_npu_w4a8_family_config {
    rk_npu_w4a8_autotune_config base; /* M ignored */
    int m_count;
    const int *m_values;
    const double *frequencies;        /* relative call counts; NULL = equal */
} rk_npu_w4a8_family_config;
typedef struct rk_npu_w4a8_family_summary {
    rk_npu_w4a8_weight_info weights;
    uint64_t weight_fingerprint;
    double weighted_total_us, weighted_robust_us;
} rk_npu_w4a8_family_summary;
void rk_npu_w4a8_family_config_init(rk_npu_w4a8_family_config *cfg, int N, int K, int m_count, const int *m_values);
/* Each requested summary needs a strategy array of m_count elements; cached forms keep one file per batch
 * size under cache_directory (NULL: the default location). */
int rk_npu_w4a8_autotune_family(rk_npu_ctx *ctx, const rk_npu_w4a8_family_config *cfg, const int8_t *B,
                                const float *w_scale, rk_npu_w4a8_family_summary *fastest,
                                rk_npu_w4a8_strategy *fastest_strategies, rk_npu_w4a8_family_summary *stable,
                                rk_npu_w4a8_strategy *stable_strategies);
int rk_npu_w4a8_autotune_family_cached(rk_npu_ctx *ctx, const rk_npu_w4a8_family_config *cfg, const int8_t *B,
                                       const float *w_scale, const char *cache_directory, int refresh,
                                       rk_npu_w4a8_family_summary *fastest, rk_npu_w4a8_strategy *fastest_strategies,
                                       rk_npu_w4a8_family_summary *stable, rk_npu_w4a8_strategy *stable_strategies,
                                       int *cache_hits, int *cache_misses);
int rk_npu_w4a8_autotune_family_ex(rk_npu_ctx *ctx, const rk_npu_w4a8_family_config *cfg, const int8_t *B,
                                   const float *w_scale, rk_npu_w4a8_family_summary *fastest,
                                   rk_npu_w4a8_strategy_ex *fastest_strategies, rk_npu_w4a8_family_summary *stable,
                                   rk_npu_w4a8_strategy_ex *stable_strategies);
int rk_npu_w4a8_autotune_family_cached_ex(rk_npu_ctx *ctx, const rk_npu_w4a8_family_config *cfg, const int8_t *B,
                                          const float *w_scale, const char *cache_directory, int refresh,
                                          rk_npu_w4a8_family_summary *fastest, rk_npu_w4a8_strategy_ex *fastest_strategies,
                                          rk_npu_w4a8_family_summary *stable, rk_npu_w4a8_strategy_ex *stable_strategies,
                                          int *cache_hits, int *cache_misses);

#ifdef __cplusplus
}
#endif
#endif /* RKNPU_B200_W4A8_H */
