/* rknpu_b200_rmsnorm.h -- the original project's residual add + RMSNorm header (include/rk_npu_add_rmsnorm_f16.h) as
 * this library implements it: the step that precedes the quantised FFN in a decoder layer.
 *
 *   residual_out = fp16(x + residual)                         the fp32 sum of the two fp16 values, rounded once more
 *   norm_out     = fp16(residual_out / sqrt(mean(residual_out^2) + eps) * gamma)
 *
 * The original runs fixed register programs on its NPU and states its result through its board test
 * (tests/test_add_rmsnorm_f16.cpp:96-127): residual_out must equal the expression above bit for bit, norm_out must be
 * within 0.04 (cosine >= 0.99999) of the double-precision evaluation "sum of squares in double, inv = 1 / sqrt(sum / D
 * + eps), fp16(float(double(v) * inv * double(gamma)))".  This library evaluates that double-precision expression;
 * the squares are added in a fixed tree order instead of one after the other, so the sum can differ from the
 * sequential one in its last bits (about 1e-16 relative), which moves an fp16 output only if a product lies that close
 * to a rounding boundary.  The order is fixed by the shape (rows, D), not by the schedule: the same call gives the same
 * bits every time.
 * The original accepts M = 1 or 128, D = 4096, eps = 1e-5 only (its validated programs); this library accepts those and
 * every 1 <= M <= 65536, D a multiple of 8 in 8..32768, eps finite and >= 0.
 * Programs may include the original header instead of this one; names, layouts and values are the same.
 */
#ifndef RKNPU_B200_RMSNORM_H
#define RKNPU_B200_RMSNORM_H
#include "rknpu_b200_w4a8.h"
#ifdef __cplusplus
extern "C" {
#endif

/* include/rk_npu_add_rmsnorm_f16.h:11-16 */
typedef struct {
    int M;
    int D;
    float eps;
    uint32_t timeout_ms; /* carried; a launch here cannot wait on anything */
} rk_npu_add_rmsnorm_f16_config;

/* include/rk_npu_add_rmsnorm_f16.h:18-25.  Filled here: tensor_bytes = 2 M D; weight_bytes = 2 D (gamma in device
 * memory); num_tasks = 1 (one launch); the other fields describe the original device's command buffers and are 0. */
typedef struct {
    uint64_t tensor_bytes;
    uint64_t internal_bytes;
    uint64_t weight_bytes;
    uint64_t regcmd_bytes;
    uint64_t task_bytes;
    int num_tasks;
} rk_npu_add_rmsnorm_f16_sizes;

typedef struct rk_npu_add_rmsnorm_f16_plan rk_npu_add_rmsnorm_f16_plan;

/* include/rk_npu_add_rmsnorm_f16.h:29-35: M, D as given, eps = 1e-5, timeout_ms = 6000.  query: RK_NPU_ERR_PARAM for
 * NULL or a configuration outside the ranges above. */
void rk_npu_add_rmsnorm_f16_config_init(rk_npu_add_rmsnorm_f16_config *cfg, int M, int D);
int rk_npu_add_rmsnorm_f16_query(const rk_npu_add_rmsnorm_f16_config *cfg, rk_npu_add_rmsnorm_f16_sizes *out);

/* include/rk_npu_add_rmsnorm_f16.h:37-41: gamma[D], fp16 bit patterns, is copied into the plan. */
rk_npu_add_rmsnorm_f16_plan *rk_npu_add_rmsnorm_f16_plan_create(rk_npu_iommu_domain *domain,
                                                                const rk_npu_add_rmsnorm_f16_config *cfg,
                                                                const uint16_t *gamma);

/* include/rk_npu_add_rmsnorm_f16.h:43-50.  All four are buffers from rk_npu_mem_alloc (or views) holding the tensor in
 * the original's block-8 layout (D/8, M, 8): element (m, d) at ((d / 8) * M + m) * 8 + d % 8.  Blocking.
 * RK_NPU_ERR_PARAM: NULL, a plan of another context, an output that overlaps an input or the other output;
 * RK_NPU_ERR_NOMEM: a buffer of another context or smaller than 2 M D bytes; RK_NPU_ERR_DOMAIN: a buffer of another
 * domain; RK_NPU_ERR_BUSY: the plan is running another call; RK_NPU_ERR_SUBMIT: the launch failed. */
int rk_npu_add_rmsnorm_f16_run(rk_npu_ctx *ctx, rk_npu_add_rmsnorm_f16_plan *plan, const rk_npu_mem *x_native,
                               const rk_npu_mem *residual_native, rk_npu_mem *residual_out_native,
                               rk_npu_mem *norm_out_native);

void rk_npu_add_rmsnorm_f16_plan_free(rk_npu_add_rmsnorm_f16_plan *plan);

#ifdef __cplusplus
}
#endif
#endif
