/* rknpu_b200_quant.h -- the part of the original project's second public header
 * (include/rk_npu_quant_matmul.h) and of include/rk_npu_matmul_i4.h that the W4A8 path's
 * callers touch: the load-only W8 tuning cache and the configuration initialisers.
 *
 * Every other entry point of those two headers (W8A8 weights / workspaces / runs, the exact
 * int4 x int4 -> int32 API, the W8 search tuners and their family forms, cache saving of
 * the W8 tuner, the DMA-buffer helpers of rk_npu_common.h) is exported by the library so that
 * existing programs link, and answers RK_NPU_ERR_PARAM, NULL or 0: those operators are not
 * built here.  Programs may include the original headers instead of this one; the layouts
 * below are the same.
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
/* Load-only W8 tuning cache (src/rk_npu_quant_matmul.cpp:183-349,1552-1563): reads one cache
 * file written by the original tuner, checks magic, key (format 2, tuning revision 6 with the
 * execution mode in its upper half, driver version of ctx, operator, shape, permission masks
 * intersected with the process affinity, measurement settings, required K tile) and both
 * records, and returns them.  RK_NPU_ERR_CACHE_MISS for an absent, malformed, stale or
 * foreign file -- and for records that name a panel layout, whose device-specific geometry
 * rules are not restated here; RK_NPU_ERR_PARAM for bad arguments. */
int rk_npu_matmul_autotune_cache_load(rk_npu_ctx *ctx, const char *cache_path, rk_npu_matmul_op_kind kind,
                                      const rk_npu_matmul_autotune_config *cfg, rk_npu_matmul_strategy *fastest,
                                      rk_npu_matmul_strategy *stable);

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

#ifdef __cplusplus
}
#endif
#endif /* RKNPU_B200_QUANT_H */
