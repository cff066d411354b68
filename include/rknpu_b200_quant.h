/* rknpu_b200_quant.h -- the original project's second public header (include/rk_npu_quant_matmul.h) as this
 * library implements it, plus the configuration initialiser of include/rk_npu_matmul_i4.h.
 *
 * Built: the typed W8A8 operators with raw int8 weights (weight objects, workspaces made from a strategy, the
 * blocking run calls, the memory queries, the K-partition query), the W8 tuning cache files (load and save), the exact
 * int4 x int4 -> int32 operator of include/rk_npu_matmul_i4.h (with its producer callback) and the configuration
 * initialisers.
 * The *_weights_create_compress constructors (include/rk_npu_quant_matmul.h:321-330,348-350,392-394: lossless
 * compressed storage of the same B for the original device's hardware decompressor, same run and free functions, same
 * results) make ordinary weight objects here: the codes are stored as they are, nothing is encoded and no memory is
 * saved; rk_npu_f32i8f32_weights_compressed_layout_generation is 0 for them, as for every uncompressed object.
 * Exported but declined (RK_NPU_ERR_PARAM, NULL or 0, nothing else happens): the W8 search tuners and their family
 * forms; the *_create_from_f32_compress constructors, which search a quantisation under a size
 * budget measured in the original device's compressed format.
 * Programs may include the original headers instead of this one; names, layouts and values are the same.
 */
#ifndef RKNPU_B200_QUANT_H
#define RKNPU_B200_QUANT_H
#include "rknpu_b200_w4a8.h"
#ifdef __cplusplus
extern "C" {
#endif

/* Operator a W8 tuning record belongs to (include/rk_npu_quant_matmul.h:44-50). */
typedef enum rk_npu_matmul_op_kind {
    RK_NPU_MATMUL_I8I8I32 = 0,
    RK_NPU_MATMUL_F16I8F16_DYNAMIC = 1,
    RK_NPU_MATMUL_F16I8F16_STATIC = 2,
    RK_NPU_MATMUL_F32I8F32_DYNAMIC = 3,
    RK_NPU_MATMUL_F32I8F32_STATIC = 4,
} rk_npu_matmul_op_kind;
/* Layout recipes a record may name (include/rk_npu_quant_matmul.h:52-66).  They describe the
 * original device's execution; here they are validated and carried, nothing else. */
typedef enum rk_npu_matmul_a_layout {
    RK_NPU_MATMUL_A_LAYOUT_NORMAL = 0,
    RK_NPU_MATMUL_A_LAYOUT_NATIVE_K16_M16 = 1,
    RK_NPU_MATMUL_A_LAYOUT_PANEL8 = 2,
    RK_NPU_MATMUL_A_LAYOUT_PANEL16 = 3,
} rk_npu_matmul_a_layout;
typedef enum rk_npu_matmul_c_layout {
    RK_NPU_MATMUL_C_LAYOUT_NATIVE = 0,
    RK_NPU_MATMUL_C_LAYOUT_PANEL8 = 1,
    RK_NPU_MATMUL_C_LAYOUT_PANEL16 = 2,
} rk_npu_matmul_c_layout;

/* include/rk_npu_quant_matmul.h:68-92 */
typedef struct rk_npu_matmul_autotune_config {
    int M, N, K;
    uint32_t allowed_npu_core_mask;   /* 0 = all; subsets of 7 */
    uint64_t allowed_cpu_core_mask;   /* 0 = the process affinity */
    int warmup, loops, repeats;
    uint32_t timeout_ms;
    int verbose;
    int required_k_tile;              /* 0 = any */
} rk_npu_matmul_autotune_config;
/* include/rk_npu_quant_matmul.h:100-114 */
typedef struct rk_npu_matmul_family_autotune_config {
    int K, N;
    int m_count;
    const int *m_values;
    const double *frequencies;
    uint32_t allowed_npu_core_mask;
    uint64_t allowed_cpu_core_mask;
    int warmup, loops, repeats;
    uint32_t timeout_ms;
    int verbose;
} rk_npu_matmul_family_autotune_config;
/* include/rk_npu_quant_matmul.h:116-147 */
typedef struct rk_npu_matmul_strategy {
    rk_npu_matmul_op_kind op_kind;
    int M, N, K;
    int k_tile, n_tile;
    rk_npu_matmul_a_layout a_layout;
    int wave_count, n_groups;
    uint32_t npu_core_mask;
    uint64_t cpu_core_mask;
    int cpu_threads;
    double input_us, npu_us, sync_us, output_us, total_us, jitter_pct, robust_us;
    rk_npu_matmul_c_layout c_layout;
} rk_npu_matmul_strategy;

/* Defaults: all three cores, 2 warm-ups, 8 loops, 3 repeats, 500 ms
 * (src/rk_npu_quant_matmul.cpp:1522-1550). */
void rk_npu_matmul_autotune_config_init(rk_npu_matmul_autotune_config *cfg, int M, int N, int K);
void rk_npu_matmul_family_autotune_config_init(rk_npu_matmul_family_autotune_config *cfg, int N, int K, int m_count,
                                               const int *m_values);
/* W8 tuning cache files (src/rk_npu_quant_matmul.cpp:183-349,1552-1579), the original's format byte for byte in both
 * directions.  load reads one file, checks magic, key (format 2, tuning revision 6 with the execution mode in its
 * upper half, driver version of ctx, operator, shape, permission masks intersected with the process affinity,
 * measurement settings, required K tile) and both records, and returns them: RK_NPU_ERR_CACHE_MISS for an absent,
 * malformed, stale or foreign file or a record the original would not accept (records that name panel layouts are
 * checked by the original's device-plan rule); RK_NPU_ERR_PARAM for bad arguments.  save checks the two strategies
 * against the same key and rules (RK_NPU_ERR_PARAM) and writes the file under a temporary name, renamed over the target
 * when complete (RK_NPU_ERR_IO).  The search that would fill such a file on this library is not built: the strategies
 * come from the caller (for instance from a file made on the original board). */
int rk_npu_matmul_autotune_cache_load(rk_npu_ctx *ctx, const char *cache_path, rk_npu_matmul_op_kind kind,
                                      const rk_npu_matmul_autotune_config *cfg, rk_npu_matmul_strategy *fastest,
                                      rk_npu_matmul_strategy *stable);
int rk_npu_matmul_autotune_cache_save(rk_npu_ctx *ctx, const char *cache_path, rk_npu_matmul_op_kind kind,
                                      const rk_npu_matmul_autotune_config *cfg, const rk_npu_matmul_strategy *fastest,
                                      const rk_npu_matmul_strategy *stable);

/* ---------------------------------------------------------------- typed W8A8 operators
 * include/rk_npu_quant_matmul.h:94-99,149-176,186-188,296-421.  int8 B[K,N] (symmetric, zero point 0) with one
 * positive scale per output channel; A and C are compact row-major host tensors (device pointers are accepted too)
 * handed to blocking calls.
 *
 *   dynamic   a_scale[m] = max|A[m,:]| / 127 (all-zero row -> 1; no lower clamp, NaN never raises the maximum)
 *   static    a_scale[m] given by the caller, finite and positive
 *   codes     clamp(round_half_away(A[m,k] * (1 / a_scale[m])), -127, 127)
 *   C[m,n]    (float(sum_k code * B) * a_scale[m]) * w_scale[n], rounded once more for binary16
 *   i8i8i32   no quantisation; sums are exact modulo 2^32
 * (src/rk_npu_cpu_kernels.cpp:126-131,576-660,853-871,1312).  Unlike the W4A8 path these operators do not reject
 * non-finite activations: they propagate as in the original's scalar code.
 *
 * On this library the contraction runs on the tcgen05 per-tile kernel with int8 weights in tensor memory.  A
 * strategy's tile, layout and mask fields are validated as the original validates them and otherwise carry no
 * meaning here; k_tile stays the compatibility key between a workspace and its weights.  Contexts opened as a
 * rank of a group of GPUs do not create these objects. */
typedef struct rk_npu_matmul_weight_config {
    int K;
    int N;
    int k_tile;
} rk_npu_matmul_weight_config;
typedef struct rk_npu_matmul_workspace_requirements {
    uint64_t bytes;           /* all device memory of the workspace */
    uint64_t input_bytes;     /* activation codes and the staged copy of A */
    uint64_t output_bytes;    /* the staged copy of C */
    uint64_t control_bytes;   /* scales and the status block */
    uint32_t wave_count;      /* ceil(K / k_tile), as the original reports it */
    uint32_t buffer_count;
} rk_npu_matmul_workspace_requirements;
typedef struct rk_npu_matmul_weight_requirements {
    uint64_t bytes;
    uint64_t packed_b_bytes;
    uint64_t scale_bytes;
    uint32_t wave_count;
    uint32_t buffer_count;
} rk_npu_matmul_weight_requirements;
typedef struct rk_npu_i8i8i32_weights rk_npu_i8i8i32_weights;
typedef struct rk_npu_f16i8f16_weights rk_npu_f16i8f16_weights;
typedef struct rk_npu_f32i8f32_weights rk_npu_f32i8f32_weights;
typedef struct rk_npu_matmul_workspace rk_npu_matmul_workspace;

/* The original tuner's conservative K-partition policy, a pure function (src/rk_npu_quant_matmul.cpp:1131-1142,
 * 1696-1700): OK for an eligible partition, PARAM otherwise. */
int rk_npu_matmul_k_partition_query(int M, int K, int k_tile);
int rk_npu_matmul_workspace_memory_query(const rk_npu_matmul_strategy *strategy, rk_npu_matmul_workspace_requirements *out);
int rk_npu_i8i8i32_weights_memory_query(const rk_npu_matmul_weight_config *config, rk_npu_matmul_weight_requirements *out);
int rk_npu_f16i8f16_weights_memory_query(const rk_npu_matmul_weight_config *config, rk_npu_matmul_weight_requirements *out);
int rk_npu_f32i8f32_weights_memory_query(const rk_npu_matmul_weight_config *config, rk_npu_matmul_weight_requirements *out);
/* Fixed to one exact M and operator; non-reentrant (concurrent use returns BUSY); NULL for an invalid strategy. */
rk_npu_matmul_workspace *rk_npu_matmul_workspace_create(rk_npu_iommu_domain *domain, const rk_npu_matmul_strategy *strategy);
void rk_npu_matmul_workspace_free(rk_npu_matmul_workspace *workspace);

rk_npu_i8i8i32_weights *rk_npu_i8i8i32_weights_create(rk_npu_iommu_domain *domain, const rk_npu_matmul_weight_config *config,
                                                      const int8_t *B_rowmajor);
void rk_npu_i8i8i32_weights_free(rk_npu_i8i8i32_weights *weights);
int rk_npu_i8i8i32_run(rk_npu_matmul_workspace *workspace, const rk_npu_i8i8i32_weights *weights, const int8_t *A_rowmajor,
                       int32_t *C_rowmajor);

/* Every w_scale must be finite and positive; both inputs may be released after creation. */
rk_npu_f16i8f16_weights *rk_npu_f16i8f16_weights_create(rk_npu_iommu_domain *domain, const rk_npu_matmul_weight_config *config,
                                                        const int8_t *B_rowmajor, const float *w_scale);
void rk_npu_f16i8f16_weights_free(rk_npu_f16i8f16_weights *weights);
int rk_npu_f16i8f16_run_dynamic(rk_npu_matmul_workspace *workspace, const rk_npu_f16i8f16_weights *weights,
                                const uint16_t *A_fp16_rowmajor, uint16_t *C_fp16_rowmajor);
int rk_npu_f16i8f16_run_static(rk_npu_matmul_workspace *workspace, const rk_npu_f16i8f16_weights *weights,
                               const uint16_t *A_fp16_rowmajor, const float *a_scale, uint16_t *C_fp16_rowmajor);

rk_npu_f32i8f32_weights *rk_npu_f32i8f32_weights_create(rk_npu_iommu_domain *domain, const rk_npu_matmul_weight_config *config,
                                                        const int8_t *B_rowmajor, const float *w_scale);
void rk_npu_f32i8f32_weights_free(rk_npu_f32i8f32_weights *weights);
/* The compressed-storage constructors: the same objects as the plain ones here (see the head of this file). */
rk_npu_i8i8i32_weights *rk_npu_i8i8i32_weights_create_compress(rk_npu_iommu_domain *domain, const rk_npu_matmul_weight_config *config,
                                                               const int8_t *B_rowmajor);
rk_npu_f16i8f16_weights *rk_npu_f16i8f16_weights_create_compress(rk_npu_iommu_domain *domain, const rk_npu_matmul_weight_config *config,
                                                                 const int8_t *B_rowmajor, const float *w_scale);
rk_npu_f32i8f32_weights *rk_npu_f32i8f32_weights_create_compress(rk_npu_iommu_domain *domain, const rk_npu_matmul_weight_config *config,
                                                                 const int8_t *B_rowmajor, const float *w_scale);
uint64_t rk_npu_f32i8f32_weights_compressed_layout_generation(const rk_npu_f32i8f32_weights *weights);
int rk_npu_f32i8f32_run_dynamic(rk_npu_matmul_workspace *workspace, const rk_npu_f32i8f32_weights *weights,
                                const float *A_fp32_rowmajor, float *C_fp32_rowmajor);
int rk_npu_f32i8f32_run_static(rk_npu_matmul_workspace *workspace, const rk_npu_f32i8f32_weights *weights,
                               const float *A_fp32_rowmajor, const float *a_scale, float *C_fp32_rowmajor);
/* No counterpart in the original: kernels this workspace has launched so far (tests use it to see that the
 * CUDA path ran). */
uint64_t rk_npu_b200_matmul_launch_count(const rk_npu_matmul_workspace *workspace);

/* include/rk_npu_matmul_i4.h:26-35; defaults m_tile 128, k_tile 480, n_tile 1024, core mask 1,
 * 500 ms, pipelined, one CPU thread (src/rk_npu_matmul_i4.cpp:10-12). */
typedef struct rk_npu_i4_config {
    int M, N, K;
    int m_tile, k_tile, n_tile;
    uint32_t npu_core_mask;
    uint32_t timeout_ms;
    int pipeline;
    int cpu_threads;
} rk_npu_i4_config;
void rk_npu_i4_config_init(rk_npu_i4_config *cfg, int M, int N, int K);

/* ---------------------------------------------------------------- exact int4 x int4 -> int32 operator
 * include/rk_npu_matmul_i4.h:37-105.  Host codes are int8 elements in [-8,7]; codes outside that range are an argument
 * error, never masked.  C is compact row-major int32, exact.  Weights depend only on (K, N, k_tile) and may be shared by
 * workspaces of any M; a workspace is fixed-shape and non-reentrant (BUSY).  Configuration rules, the memory query's
 * figures (they describe the original device's buffers) and every return code are the original's; an explicit k_tile
 * above 480 still needs the weights to prove that no INT16 partial of the original device could saturate.  On this
 * library the sums are accumulated in int32 directly, so nothing saturates.  A and C may also be device pointers. */
typedef struct rk_npu_i4_timings {
    double pack_us;    /* host: code validation, or the producer callbacks and their decoding */
    double sync_us;    /* host-to-device copy of the activations */
    double submit_us;  /* the two kernels and the copy of C, until the stream has drained */
    double reduce_us;  /* always 0 here: there is no host reduction */
    double total_us;
} rk_npu_i4_timings;
typedef struct rk_npu_i4i4i32_weights rk_npu_i4i4i32_weights;
typedef struct rk_npu_i4_workspace rk_npu_i4_workspace;
int rk_npu_i4_memory_query(const rk_npu_i4_config *cfg, rk_npu_i4_memory_info *out);
rk_npu_i4i4i32_weights *rk_npu_i4i4i32_weights_create(rk_npu_iommu_domain *domain, const rk_npu_i4_weight_config *cfg, const int8_t *B);
void rk_npu_i4i4i32_weights_free(rk_npu_i4i4i32_weights *weights);
rk_npu_i4_workspace *rk_npu_i4_workspace_create(rk_npu_iommu_domain *domain, const rk_npu_i4_config *cfg);
void rk_npu_i4_workspace_free(rk_npu_i4_workspace *workspace);
int rk_npu_i4i4i32_run(rk_npu_i4_workspace *workspace, const rk_npu_i4i4i32_weights *weights, const int8_t *A, int32_t *C,
                       rk_npu_i4_timings *timings);
/* Fused preprocessing boundary: the producer is invoked serially on the calling thread for each K wave (k_tile) and M
 * panel (m_tile), in increasing K then M order, with a zero-initialised [padded_k / 32][rows][32] int4 tile, even element
 * in the HIGH nibble; it writes the logical codes and returns RK_NPU_OK or an error, which ends the run. */
typedef struct rk_npu_i4_input_tile {
    int m0, rows, k0, k, padded_k;
    uint8_t *dst;
    uint64_t bytes;
} rk_npu_i4_input_tile;
typedef int (*rk_npu_i4_input_producer)(void *user, const rk_npu_i4_input_tile *tile);
int rk_npu_i4i4i32_run_with_producer(rk_npu_i4_workspace *workspace, const rk_npu_i4i4i32_weights *weights,
                                     rk_npu_i4_input_producer producer, void *user, int32_t *C, rk_npu_i4_timings *timings);
/* The reference producer: packs rows [m0, m0 + rows) x columns [k0, k0 + k) of A (leading dimension lda) into the tile. */
int rk_npu_i4_pack_a_tile(const rk_npu_i4_input_tile *tile, const int8_t *A, int lda);

#ifdef __cplusplus
}
#endif
#endif /* RKNPU_B200_QUANT_H */
