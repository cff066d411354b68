/* rknpu_b200_moe.h -- the original project's routed-experts header (include/rk_npu_moe_w8.h) as this library
 * implements it: routed SwiGLU experts with int8 or int4 weights plus an optional shared expert; the router is the
 * caller's.
 *
 * Built: configuration, immutable expert weight objects (int8 experts; int4 experts; routed int4 experts with an int8
 * shared expert), mutable slot banks of int4 experts with their cache records, workspaces of the matching form, the two blocking run calls (int8 rows with scales, or fp32 rows
 * quantised here), the byte queries.  All pointers are host pointers and a call returns when the output is complete, as
 * in the original.  Int4 experts are given as int8 arrays of codes in [-8, 7]; they are accepted under the original's
 * rule (the K tile its device would run must be certified against INT16 partial sums: the whole of K where it would try
 * that, else slices of 512) and are then stored two codes per byte; the sums are the same integers as for int8 storage.
 * Mutable slot banks (rk_npu_moe_*_slots_create) hold int4 experts that come and go as cache records: export from any
 * bank with int4 experts, import into any slot, exchange slots between two banks without a copy.
 * Exported but declined: RK_NPU_MOE_MIDDLE_NPU_LUT, the original device's approximate table-lookup activation (a
 * workspace that asks for it is not created).
 * Programs may include the original header instead of this one; names, layouts and values are the same.
 */
#ifndef RKNPU_B200_MOE_H
#define RKNPU_B200_MOE_H
#include "rknpu_b200_w4a8.h"
#ifdef __cplusplus
extern "C" {
#endif

/* include/rk_npu_moe_w8.h:14-29.  The fused fp32 middle stage (dequantise, SwiGLU with the degree-7 polynomial the
 * dense path uses, row maximum, nearest-even int8) is the only one built. */
typedef enum rk_npu_moe_middle {
    RK_NPU_MOE_MIDDLE_CPU = 0,
    RK_NPU_MOE_MIDDLE_NPU_LUT = 1
} rk_npu_moe_middle;

/* include/rk_npu_moe_w8.h:31-36 */
typedef struct rk_npu_moe_w8_weight_config {
    int hidden;         /* >= 64, multiple of 32 (this library: at most 8192) */
    int intermediate;   /* 32..512, multiple of 32 */
    int routed_experts; /* >= 1 */
    int shared_expert;  /* 0 or 1; if present, expert index routed_experts */
} rk_npu_moe_w8_weight_config;

/* include/rk_npu_moe_w8.h:38-48.  npu_cores, cpu_threads and native_input are validated and carried; they describe
 * the original device's execution and change nothing here. */
typedef struct rk_npu_moe_w8_config {
    uint32_t struct_size;
    rk_npu_moe_w8_weight_config weights;
    int max_rows;      /* 1..256; each run may use any smaller positive count */
    int top_k;         /* 1..min(routed_experts, 8) */
    int npu_cores;     /* 1/2/3 */
    int cpu_threads;   /* 1..4 */
    int native_input;  /* 0 or 1 */
    rk_npu_moe_middle middle;
    uint32_t timeout_ms;
} rk_npu_moe_w8_config;

/* include/rk_npu_moe_w8.h:50-57: compact signed int8, gate columns followed by up columns; copied at creation. */
typedef struct rk_npu_moe_w8_expert {
    const int8_t* gate_up;       /* [hidden, 2*intermediate] */
    const float* gate_up_scales; /* [2*intermediate], positive finite */
    const int8_t* down;          /* [intermediate, hidden] */
    const float* down_scales;    /* [hidden], positive finite */
} rk_npu_moe_w8_expert;

/* include/rk_npu_moe_w8.h:59-65.  Filled here: input_us (upload and quantisation), schedule_us (grouping the routes on
 * the host), gate_us / down_us / combine_us (the three launches, device time), sync_us (result download and wait),
 * total_us, gemm_tasks (jobs of at most 16 assignments), gather_tasks = middle_tasks = assignments. */
typedef struct rk_npu_moe_w8_timings {
    double input_us, schedule_us, build_us, sync_us, gather_us;
    double gate_us, middle_npu_us, middle_cpu_us, down_us, combine_us;
    double lut_load_us;
    double total_us;
    uint32_t gather_tasks, middle_tasks, gemm_tasks;
} rk_npu_moe_w8_timings;

typedef struct rk_npu_moe_w8_weights rk_npu_moe_w8_weights;
typedef struct rk_npu_moe_w8_workspace rk_npu_moe_w8_workspace;

/* include/rk_npu_moe_w8.h:70-74 */
void rk_npu_moe_w8_config_init(rk_npu_moe_w8_config* config, int hidden, int intermediate, int routed_experts,
                               int shared_expert, int top_k, int max_rows);

/* include/rk_npu_moe_w8.h:76-85.  NULL for an invalid configuration, a NULL array, a scale that is not positive and
 * finite, or a failed allocation. */
rk_npu_moe_w8_weights* rk_npu_moe_w8_weights_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                    const rk_npu_moe_w8_expert* experts);
void rk_npu_moe_w8_weights_free(rk_npu_moe_w8_weights* weights);
rk_npu_moe_w8_workspace* rk_npu_moe_w8_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_config* config);
void rk_npu_moe_w8_workspace_free(rk_npu_moe_w8_workspace* workspace);

/* include/rk_npu_moe_w8.h:148-152: device payload bytes of a handle; a slot bank counts the slots it holds now. */
uint64_t rk_npu_moe_w8_weights_device_bytes(const rk_npu_moe_w8_weights* weights);
uint64_t rk_npu_moe_w8_workspace_device_bytes(const rk_npu_moe_w8_workspace* workspace);

/* include/rk_npu_moe_w8.h:154-177.  expert_ids / route_weights are row-major [rows, top_k]; ids in [0, routed_experts),
 * coefficients finite and >= 0; duplicates are summed in slot order; a zero coefficient leaves the route out; the shared
 * expert is appended with coefficient 1; no normalisation.  Output: compact fp32 [rows, hidden].
 * run_quantized: int8 [rows, hidden] with one positive finite scale per row, used as given.  run_f32: rows quantised
 * once with nearest-even rounding and scale max/127 (1 for a zero row).
 * RK_NPU_ERR_PARAM: NULL / rows out of range / overlapping arrays / bad id, coefficient, scale or non-finite input /
 * weights of another geometry; RK_NPU_ERR_DOMAIN: weights of another context or domain; RK_NPU_ERR_BUSY: workspace in
 * use.  A rejected call does not write the output. */
int rk_npu_moe_w8_run_quantized(rk_npu_moe_w8_workspace* workspace, const rk_npu_moe_w8_weights* weights, int rows,
                                const int8_t* input, const float* row_scales, const int32_t* expert_ids,
                                const float* route_weights, float* output, rk_npu_moe_w8_timings* timings);
int rk_npu_moe_w8_run_f32(rk_npu_moe_w8_workspace* workspace, const rk_npu_moe_w8_weights* weights, int rows,
                          const float* input, const int32_t* expert_ids, const float* route_weights, float* output,
                          rk_npu_moe_w8_timings* timings);

/* include/rk_npu_moe_w8.h:87-111: all experts int4 (..._quant_...; _full_k also tries the whole of K for gate/up), or
 * routed int4 experts with an int8 shared expert (..._w4_...).  hidden and intermediate multiples of 64, hidden <= 8128,
 * normal input; NULL when a code is outside [-8, 7] or the tile cannot be certified.  The handles use the run / free /
 * byte-query functions above; a workspace runs weights of its own form only (RK_NPU_ERR_PARAM otherwise). */
rk_npu_moe_w8_weights* rk_npu_moe_quant_weights_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                       const rk_npu_moe_w8_expert* experts);
rk_npu_moe_w8_weights* rk_npu_moe_quant_weights_create_full_k(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                              const rk_npu_moe_w8_expert* experts);
rk_npu_moe_w8_workspace* rk_npu_moe_quant_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_config* config);
rk_npu_moe_w8_weights* rk_npu_moe_w4_weights_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                    const rk_npu_moe_w8_expert* experts);
rk_npu_moe_w8_workspace* rk_npu_moe_w4_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_config* config);
/* ---- mutable slot banks and cache records: include/rk_npu_moe_w8.h:113-146
 * A slot bank has the geometry of a weight object but no experts yet: every slot is imported before it is selected (an
 * empty slot contributes zero).  rk_npu_moe_quant_slots_create: all slots int4 experts (shared_expert must be 0);
 * rk_npu_moe_w4_slots_create: routed int4 slots plus the immutable int8 shared expert given here (shared_expert must
 * be 1).  The caller owns the mapping of logical experts to slots.  A slot bank runs with the workspace of its form
 * (quant / w4) like any other weight object.
 *
 * A cache record is one int4 expert in this library's execution layout: gate/up records, down records, the two scale
 * arrays, and a 16-byte trailer (magic, hidden, intermediate, and in the low three bits of the LAST 32-bit word the
 * original's tag: 1 = gate/up certified in slices, 2 = over the whole of K).  rk_npu_moe_quant_expert_blob_bytes is its
 * size (0 for a bank without int4 experts); buffers may be larger (a file store can page-align its stride).  Records of
 * the same expert exported from an immutable all-int4 bank, a whole-K certified one, the mixed form or a slot are the
 * same bytes.  They are NOT the original device's records: a cache written on the original board is refused by the
 * trailer check.
 * export: RK_NPU_ERR_PARAM for NULL, a short buffer, an index out of range or the int8 shared expert.
 * import: additionally RK_NPU_ERR_PARAM for a foreign or untagged trailer, another geometry, a whole-K tag where hidden
 * does not allow it, or a scale that is not positive and finite; the record is checked before anything is copied, so a
 * refused record leaves the slot as it was.  Import only between blocking runs that use the bank; imports into
 * different slots, and into a bank that is not running, may overlap runs and each other.  _timed fills validate_us,
 * gate_sync_us (the transfer; for an immutable bank the gate/up part) and down_sync_us, total_us; copy_us stays 0.
 * swap: exchanges the storage and tags of two slots of two all-int4 SLOT banks of one geometry, context and domain --
 * no copy, no wait; storage ownership follows the slot, either bank may be freed afterwards.  RK_NPU_ERR_PARAM
 * otherwise (the original also accepts its immutable all-int4 banks, whose experts are separate allocations there). */
rk_npu_moe_w8_weights* rk_npu_moe_w4_slots_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                  const rk_npu_moe_w8_expert* shared);
rk_npu_moe_w8_weights* rk_npu_moe_quant_slots_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config);
uint64_t rk_npu_moe_quant_expert_blob_bytes(const rk_npu_moe_w8_weights* weights);
int rk_npu_moe_quant_export_expert(const rk_npu_moe_w8_weights* weights, int expert, void* data, uint64_t bytes);
int rk_npu_moe_quant_import_expert(rk_npu_moe_w8_weights* weights, int slot, const void* data, uint64_t bytes);
typedef struct rk_npu_moe_import_timings {
    double copy_us, validate_us, gate_sync_us, down_sync_us, total_us;
} rk_npu_moe_import_timings;
int rk_npu_moe_quant_import_expert_timed(rk_npu_moe_w8_weights* weights, int slot, const void* data, uint64_t bytes,
                                         rk_npu_moe_import_timings* timings);
int rk_npu_moe_quant_swap_slots(rk_npu_moe_w8_weights* first, int first_slot, rk_npu_moe_w8_weights* second, int second_slot);

#ifdef __cplusplus
}
#endif
#endif
