// w4a8_unbuilt.cpp -- entry points of the original project's public headers that this library
// does not implement: the W8 search tuners and their family forms, and the constructors that
// quantise under a compressed-size budget (include/rk_npu_quant_matmul.h).  They are
// exported so that programs written against those headers link and start; each one declines: RK_NPU_ERR_PARAM, NULL, or 0, and does nothing else.
// C linkage carries no parameter types, so the definitions take none; the callers' arguments
// are ignored.
#include "../../include/rknpu_b200_w4a8.h"
#include <stdint.h>

#define RKB200_DECLINE_INT(name) extern "C" int name(void) { return RK_NPU_ERR_PARAM; }
#define RKB200_DECLINE_PTR(name) extern "C" void* name(void) { return nullptr; }
#define RKB200_DECLINE_VOID(name) extern "C" void name(void) {}
#define RKB200_DECLINE_U64(name) extern "C" uint64_t name(void) { return 0; }

RKB200_DECLINE_INT(rk_npu_f16i8f16_dynamic_autotune)
RKB200_DECLINE_INT(rk_npu_f16i8f16_dynamic_autotune_family)
RKB200_DECLINE_INT(rk_npu_f16i8f16_static_autotune)
RKB200_DECLINE_INT(rk_npu_f16i8f16_static_autotune_family)
RKB200_DECLINE_INT(rk_npu_f32i8f32_dynamic_autotune)
RKB200_DECLINE_INT(rk_npu_f32i8f32_dynamic_autotune_family)
RKB200_DECLINE_INT(rk_npu_f32i8f32_static_autotune)
RKB200_DECLINE_INT(rk_npu_f32i8f32_static_autotune_family)
RKB200_DECLINE_INT(rk_npu_i8i8i32_autotune)
RKB200_DECLINE_INT(rk_npu_i8i8i32_autotune_family)
RKB200_DECLINE_INT(rk_npu_matmul_autotune_cached)
RKB200_DECLINE_INT(rk_npu_matmul_autotune_family_cached)

// constructors: no object
RKB200_DECLINE_PTR(rk_npu_f16i8f16_weights_create_from_f32_compress)
RKB200_DECLINE_PTR(rk_npu_f32i8f32_weights_create_from_f32_compress)

// destructors of objects that are never created, and setters without effect
RKB200_DECLINE_VOID(rk_npu_iommu_domain_set_reclaim)

