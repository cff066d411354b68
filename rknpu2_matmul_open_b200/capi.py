"""ctypes declarations of the library's C ABI (include/rknpu_b200_w4a8.h, rknpu_b200_quant.h, rknpu_b200_ext.h).

The structures below have the field order and types of the C structs one for one, so
Python code reads like a C caller of the original rk_npu_w4a8 interface.  Loading fails
loudly when the shared library has not been built; there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "librk_npu_matmul_b200.so"

RK_NPU_OK = 0
RK_NPU_ERR_OPEN = -1
RK_NPU_ERR_IOCTL = -2
RK_NPU_ERR_PARAM = -3
RK_NPU_ERR_NOMEM = -4
RK_NPU_ERR_SUBMIT = -5
RK_NPU_ERR_BUSY = -6
RK_NPU_ERR_DOMAIN = -7
RK_NPU_ERR_IO = -8
RK_NPU_ERR_CACHE_MISS = -9

RK_NPU_W4A8_SERIAL, RK_NPU_W4A8_PIPELINED, RK_NPU_W4A8_CHAIN = 0, 1, 2
RK_NPU_W4A8_INPUT_NATIVE, RK_NPU_W4A8_INPUT_PANEL8 = 0, 1
RK_NPU_W4A8_REDUCE_CPU, RK_NPU_W4A8_REDUCE_NPU = 0, 1
RK_NPU_W4A8_F32, RK_NPU_W4A8_F16 = 0, 1


class DomainMemoryStats(C.Structure):
    _fields_ = [("live_bytes", C.c_uint64), ("peak_bytes", C.c_uint64), ("creates", C.c_uint64),
                ("destroys", C.c_uint64)]


class I4WeightConfig(C.Structure):
    _fields_ = [("K", C.c_int), ("N", C.c_int), ("k_tile", C.c_int)]


class I4MemoryInfo(C.Structure):
    _fields_ = [("packed_weight_bytes", C.c_uint64), ("input_bytes", C.c_uint64), ("partial_bytes", C.c_uint64),
                ("control_bytes", C.c_uint64), ("wave_count", C.c_uint32), ("tasks_per_wave", C.c_uint32)]


class W4A8Config(C.Structure):
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("m_tile", C.c_int), ("k_tile", C.c_int),
                ("n_tile", C.c_int), ("npu_core_mask", C.c_uint32), ("timeout_ms", C.c_uint32),
                ("pipeline", C.c_int), ("cpu_threads", C.c_int)]


class W4A8MemoryInfo(C.Structure):
    _fields_ = [("backend", I4MemoryInfo), ("weight_metadata_bytes", C.c_uint64), ("cpu_scratch_bytes", C.c_uint64)]


class W4A8Options(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("input_layout", C.c_int), ("reduce_backend", C.c_int)]


class W4A8MemoryInfoEx(C.Structure):
    _fields_ = [("base", W4A8MemoryInfo), ("reduction_output_bytes", C.c_uint64),
                ("reduction_weight_bytes", C.c_uint64), ("reduction_control_bytes", C.c_uint64),
                ("workspace_bytes", C.c_uint64), ("effective_reduce_backend", C.c_int)]


class W4A8Timings(C.Structure):
    _fields_ = [("activation_scan_us", C.c_double), ("quant_pack_us", C.c_double), ("sync_us", C.c_double),
                ("submit_us", C.c_double), ("reduce_us", C.c_double), ("dequant_us", C.c_double),
                ("total_us", C.c_double)]


class W4A8FfnTimings(C.Structure):
    _fields_ = [("gate_up", W4A8Timings), ("down", W4A8Timings), ("total_us", C.c_double)]


class W4A8WeightInfo(C.Structure):
    _fields_ = [("config", I4WeightConfig), ("safe_k_tile", C.c_int), ("multiplier", C.c_double),
                ("bound_relaxed", C.c_int)]


class W4A8AutotuneConfig(C.Structure):
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("activation_type", C.c_int),
                ("allowed_npu_core_mask", C.c_uint32), ("allowed_cpu_core_mask", C.c_uint64), ("warmup", C.c_int),
                ("loops", C.c_int), ("repeats", C.c_int), ("timeout_ms", C.c_uint32), ("verbose", C.c_int),
                ("required_k_tile", C.c_int), ("k_tile_multiplier", C.c_double)]


class W4A8Strategy(C.Structure):
    _fields_ = [("config", W4A8Config), ("activation_type", C.c_int), ("cpu_core_mask", C.c_uint64),
                ("weights", W4A8WeightInfo), ("weight_fingerprint", C.c_uint64), ("tuning_revision", C.c_uint32),
                ("input_us", C.c_double), ("npu_us", C.c_double), ("sync_us", C.c_double), ("output_us", C.c_double),
                ("total_us", C.c_double), ("jitter_pct", C.c_double), ("robust_us", C.c_double)]


class MatmulAutotuneConfig(C.Structure):
    """rk_npu_matmul_autotune_config (include/rknpu_b200_quant.h): request key of the W8 tuning cache."""
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("allowed_npu_core_mask", C.c_uint32),
                ("allowed_cpu_core_mask", C.c_uint64), ("warmup", C.c_int), ("loops", C.c_int), ("repeats", C.c_int),
                ("timeout_ms", C.c_uint32), ("verbose", C.c_int), ("required_k_tile", C.c_int)]


class MatmulFamilyAutotuneConfig(C.Structure):
    _fields_ = [("K", C.c_int), ("N", C.c_int), ("m_count", C.c_int), ("m_values", C.POINTER(C.c_int)),
                ("frequencies", C.POINTER(C.c_double)), ("allowed_npu_core_mask", C.c_uint32),
                ("allowed_cpu_core_mask", C.c_uint64), ("warmup", C.c_int), ("loops", C.c_int), ("repeats", C.c_int),
                ("timeout_ms", C.c_uint32), ("verbose", C.c_int)]


class MatmulStrategy(C.Structure):
    """rk_npu_matmul_strategy: one record of the W8 tuning cache."""
    _fields_ = [("op_kind", C.c_int), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("k_tile", C.c_int),
                ("n_tile", C.c_int), ("a_layout", C.c_int), ("wave_count", C.c_int), ("n_groups", C.c_int),
                ("npu_core_mask", C.c_uint32), ("cpu_core_mask", C.c_uint64), ("cpu_threads", C.c_int),
                ("input_us", C.c_double), ("npu_us", C.c_double), ("sync_us", C.c_double), ("output_us", C.c_double),
                ("total_us", C.c_double), ("jitter_pct", C.c_double), ("robust_us", C.c_double), ("c_layout", C.c_int)]


class MatmulWeightConfig(C.Structure):
    """rk_npu_matmul_weight_config: the (K, N, k_tile) key of a W8 weight object."""
    _fields_ = [("K", C.c_int), ("N", C.c_int), ("k_tile", C.c_int)]


class MoeWeightConfig(C.Structure):
    """rk_npu_moe_w8_weight_config"""
    _fields_ = [("hidden", C.c_int), ("intermediate", C.c_int), ("routed_experts", C.c_int), ("shared_expert", C.c_int)]


class MoeConfig(C.Structure):
    """rk_npu_moe_w8_config"""
    _fields_ = [("struct_size", C.c_uint32), ("weights", MoeWeightConfig), ("max_rows", C.c_int), ("top_k", C.c_int),
                ("npu_cores", C.c_int), ("cpu_threads", C.c_int), ("native_input", C.c_int), ("middle", C.c_int),
                ("timeout_ms", C.c_uint32)]


class MoeExpert(C.Structure):
    """rk_npu_moe_w8_expert: host arrays of one expert"""
    _fields_ = [("gate_up", C.c_void_p), ("gate_up_scales", C.c_void_p), ("down", C.c_void_p), ("down_scales", C.c_void_p)]


class MoeTimings(C.Structure):
    """rk_npu_moe_w8_timings"""
    _fields_ = [(n, C.c_double) for n in ("input_us", "schedule_us", "build_us", "sync_us", "gather_us", "gate_us", "middle_npu_us",
                                          "middle_cpu_us", "down_us", "combine_us", "lut_load_us", "total_us")] + \
               [(n, C.c_uint32) for n in ("gather_tasks", "middle_tasks", "gemm_tasks")]


class Mem(C.Structure):
    """rk_npu_mem"""
    _fields_ = [("handle", C.c_uint32), ("flags", C.c_uint32), ("obj_addr", C.c_uint64), ("dma_addr", C.c_uint64),
                ("vaddr", C.c_void_p), ("size", C.c_uint64), ("offset", C.c_uint64), ("capacity", C.c_uint64),
                ("ctx_id", C.c_uint64), ("iommu_domain_id", C.c_uint32), ("reserved", C.c_uint32)]


class AddRmsNormConfig(C.Structure):
    """rk_npu_add_rmsnorm_f16_config"""
    _fields_ = [("M", C.c_int), ("D", C.c_int), ("eps", C.c_float), ("timeout_ms", C.c_uint32)]


class AddRmsNormSizes(C.Structure):
    """rk_npu_add_rmsnorm_f16_sizes"""
    _fields_ = [("tensor_bytes", C.c_uint64), ("internal_bytes", C.c_uint64), ("weight_bytes", C.c_uint64),
                ("regcmd_bytes", C.c_uint64), ("task_bytes", C.c_uint64), ("num_tasks", C.c_int)]


class MoeImportTimings(C.Structure):
    """rk_npu_moe_import_timings"""
    _fields_ = [(n, C.c_double) for n in ("copy_us", "validate_us", "gate_sync_us", "down_sync_us", "total_us")]


class MatmulWorkspaceRequirements(C.Structure):
    _fields_ = [("bytes", C.c_uint64), ("input_bytes", C.c_uint64), ("output_bytes", C.c_uint64), ("control_bytes", C.c_uint64),
                ("wave_count", C.c_uint32), ("buffer_count", C.c_uint32)]


class MatmulWeightRequirements(C.Structure):
    _fields_ = [("bytes", C.c_uint64), ("packed_b_bytes", C.c_uint64), ("scale_bytes", C.c_uint64), ("wave_count", C.c_uint32),
                ("buffer_count", C.c_uint32)]


class I4Config(C.Structure):
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("m_tile", C.c_int), ("k_tile", C.c_int),
                ("n_tile", C.c_int), ("npu_core_mask", C.c_uint32), ("timeout_ms", C.c_uint32), ("pipeline", C.c_int),
                ("cpu_threads", C.c_int)]


class I4Timings(C.Structure):
    _fields_ = [("pack_us", C.c_double), ("sync_us", C.c_double), ("submit_us", C.c_double), ("reduce_us", C.c_double),
                ("total_us", C.c_double)]


class I4InputTile(C.Structure):
    _fields_ = [("m0", C.c_int), ("rows", C.c_int), ("k0", C.c_int), ("k", C.c_int), ("padded_k", C.c_int),
                ("dst", C.POINTER(C.c_uint8)), ("bytes", C.c_uint64)]


I4_PRODUCER = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(I4InputTile))


class W4A8FamilyConfig(C.Structure):
    _fields_ = [("base", W4A8AutotuneConfig), ("m_count", C.c_int), ("m_values", C.POINTER(C.c_int)),
                ("frequencies", C.POINTER(C.c_double))]


class W4A8StrategyEx(C.Structure):
    _fields_ = [("base", W4A8Strategy), ("execution", W4A8Options)]


class W4A8FamilySummary(C.Structure):
    _fields_ = [("weights", W4A8WeightInfo), ("weight_fingerprint", C.c_uint64), ("weighted_total_us", C.c_double),
                ("weighted_robust_us", C.c_double)]


_P = C.c_void_p
_SIGNATURES = {
    # context, domains
    "rk_npu_open": (_P, [C.c_char_p]),
    "rk_npu_close": (None, [_P]),
    "rk_npu_iommu_domain_create": (_P, [_P, C.c_uint32]),
    "rk_npu_iommu_domain_free": (None, [_P]),
    "rk_npu_iommu_domain_id": (C.c_uint32, [_P]),
    "rk_npu_iommu_domain_memory_stats": (C.c_int, [_P, C.POINTER(DomainMemoryStats)]),
    "rk_npu_strerror": (C.c_char_p, [C.c_int]),
    # accounting
    "rk_npu_i4_weights_memory_query": (C.c_int, [C.POINTER(I4WeightConfig), C.POINTER(C.c_uint64)]),
    "rk_npu_w4a8_config_init": (None, [C.POINTER(W4A8Config), C.c_int, C.c_int, C.c_int]),
    "rk_npu_w4a8_options_init": (None, [C.POINTER(W4A8Options)]),
    "rk_npu_w4a8_memory_query": (C.c_int, [C.POINTER(W4A8Config), C.POINTER(W4A8MemoryInfo)]),
    "rk_npu_w4a8_memory_query_ex": (C.c_int, [C.POINTER(W4A8Config), C.POINTER(W4A8Options),
                                              C.POINTER(W4A8MemoryInfoEx)]),
    # weights, workspaces
    "rk_npu_w4a8_weights_create": (_P, [_P, C.POINTER(I4WeightConfig), _P, _P]),
    "rk_npu_w4a8_weights_free": (None, [_P]),
    "rk_npu_w4a8_weights_query": (C.c_int, [_P, C.POINTER(W4A8WeightInfo)]),
    "rk_npu_w4a8_workspace_create": (_P, [_P, C.POINTER(W4A8Config)]),
    "rk_npu_w4a8_workspace_create_ex": (_P, [_P, C.POINTER(W4A8Config), C.POINTER(W4A8Options)]),
    "rk_npu_w4a8_workspace_free": (None, [_P]),
    # runs
    "rk_npu_w4a8_run_f32": (C.c_int, [_P, _P, _P, _P, C.POINTER(W4A8Timings)]),
    "rk_npu_w4a8_run_f16": (C.c_int, [_P, _P, _P, _P, C.POINTER(W4A8Timings)]),
    "rk_npu_w4a8_run_swiglu_f32": (C.c_int, [_P, _P, _P, _P, C.POINTER(W4A8Timings)]),
    "rk_npu_w4a8_run_ffn_f32": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, C.POINTER(W4A8FfnTimings)]),
    # tuning cache
    "rk_npu_w4a8_tuning_profile_from_weights": (_P, [_P]),
    "rk_npu_w4a8_tuning_profile_free": (None, [_P]),
    "rk_npu_w4a8_tuning_profile_fingerprint": (C.c_uint64, [_P]),
    "rk_npu_w4a8_autotune_config_init": (None, [C.POINTER(W4A8AutotuneConfig), C.c_int, C.c_int, C.c_int]),
    "rk_npu_w4a8_autotune_cache_load_profile_ex": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, C.c_char_p,
                                                             C.POINTER(W4A8StrategyEx), C.POINTER(W4A8StrategyEx)]),
    "rk_npu_w4a8_autotune_cache_load": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, _P, C.c_char_p,
                                                  C.POINTER(W4A8Strategy), C.POINTER(W4A8Strategy)]),
    "rk_npu_w4a8_autotune_cache_save": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, _P, C.c_char_p,
                                                  C.POINTER(W4A8Strategy), C.POINTER(W4A8Strategy)]),
    "rk_npu_w4a8_autotune_cache_load_ex": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, _P, C.c_char_p,
                                                     C.POINTER(W4A8StrategyEx), C.POINTER(W4A8StrategyEx)]),
    "rk_npu_w4a8_autotune_cache_save_ex": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, _P, C.c_char_p,
                                                     C.POINTER(W4A8StrategyEx), C.POINTER(W4A8StrategyEx)]),
    "rk_npu_w4a8_weights_create_tuned": (_P, [_P, C.POINTER(W4A8Strategy), _P, _P]),
    "rk_npu_w4a8_weights_create_tuned_ex": (_P, [_P, C.POINTER(W4A8StrategyEx), _P, _P]),
    "rk_npu_w4a8_workspace_create_tuned_ex": (_P, [_P, C.POINTER(W4A8StrategyEx)]),
    # second header: W8 load-only cache and configuration initialisers (include/rknpu_b200_quant.h)
    "rk_npu_matmul_autotune_config_init": (None, [C.POINTER(MatmulAutotuneConfig), C.c_int, C.c_int, C.c_int]),
    "rk_npu_matmul_family_autotune_config_init": (None, [C.POINTER(MatmulFamilyAutotuneConfig), C.c_int, C.c_int, C.c_int,
                                                         C.POINTER(C.c_int)]),
    "rk_npu_matmul_autotune_cache_load": (C.c_int, [_P, C.c_char_p, C.c_int, C.POINTER(MatmulAutotuneConfig),
                                                    C.POINTER(MatmulStrategy), C.POINTER(MatmulStrategy)]),
    "rk_npu_matmul_autotune_cache_save": (C.c_int, [_P, C.c_char_p, C.c_int, C.POINTER(MatmulAutotuneConfig),
                                                    C.POINTER(MatmulStrategy), C.POINTER(MatmulStrategy)]),
    "rk_npu_i4_config_init": (None, [C.POINTER(I4Config), C.c_int, C.c_int, C.c_int]),
    # exact int4 x int4 -> int32 operator
    "rk_npu_i4_memory_query": (C.c_int, [C.POINTER(I4Config), C.POINTER(I4MemoryInfo)]),
    "rk_npu_i4i4i32_weights_create": (_P, [_P, C.POINTER(I4WeightConfig), _P]),
    "rk_npu_i4i4i32_weights_free": (None, [_P]),
    "rk_npu_i4_workspace_create": (_P, [_P, C.POINTER(I4Config)]),
    "rk_npu_i4_workspace_free": (None, [_P]),
    "rk_npu_i4i4i32_run": (C.c_int, [_P, _P, _P, _P, C.POINTER(I4Timings)]),
    "rk_npu_i4i4i32_run_with_producer": (C.c_int, [_P, _P, I4_PRODUCER, _P, _P, C.POINTER(I4Timings)]),
    "rk_npu_i4_pack_a_tile": (C.c_int, [C.POINTER(I4InputTile), _P, C.c_int]),
    # typed W8A8 operators
    "rk_npu_matmul_k_partition_query": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "rk_npu_matmul_workspace_memory_query": (C.c_int, [C.POINTER(MatmulStrategy), C.POINTER(MatmulWorkspaceRequirements)]),
    "rk_npu_i8i8i32_weights_memory_query": (C.c_int, [C.POINTER(MatmulWeightConfig), C.POINTER(MatmulWeightRequirements)]),
    "rk_npu_f16i8f16_weights_memory_query": (C.c_int, [C.POINTER(MatmulWeightConfig), C.POINTER(MatmulWeightRequirements)]),
    "rk_npu_f32i8f32_weights_memory_query": (C.c_int, [C.POINTER(MatmulWeightConfig), C.POINTER(MatmulWeightRequirements)]),
    "rk_npu_matmul_workspace_create": (_P, [_P, C.POINTER(MatmulStrategy)]),
    "rk_npu_matmul_workspace_free": (None, [_P]),
    "rk_npu_i8i8i32_weights_create": (_P, [_P, C.POINTER(MatmulWeightConfig), _P]),
    "rk_npu_i8i8i32_weights_free": (None, [_P]),
    "rk_npu_i8i8i32_run": (C.c_int, [_P, _P, _P, _P]),
    "rk_npu_f16i8f16_weights_create": (_P, [_P, C.POINTER(MatmulWeightConfig), _P, _P]),
    "rk_npu_f16i8f16_weights_free": (None, [_P]),
    "rk_npu_f16i8f16_run_dynamic": (C.c_int, [_P, _P, _P, _P]),
    "rk_npu_f16i8f16_run_static": (C.c_int, [_P, _P, _P, _P, _P]),
    "rk_npu_f32i8f32_weights_create": (_P, [_P, C.POINTER(MatmulWeightConfig), _P, _P]),
    "rk_npu_i8i8i32_weights_create_compress": (_P, [_P, C.POINTER(MatmulWeightConfig), _P]),
    "rk_npu_f16i8f16_weights_create_compress": (_P, [_P, C.POINTER(MatmulWeightConfig), _P, _P]),
    "rk_npu_f32i8f32_weights_create_compress": (_P, [_P, C.POINTER(MatmulWeightConfig), _P, _P]),
    "rk_npu_f32i8f32_weights_compressed_layout_generation": (C.c_uint64, [_P]),
    "rk_npu_f32i8f32_weights_free": (None, [_P]),
    "rk_npu_f32i8f32_run_dynamic": (C.c_int, [_P, _P, _P, _P]),
    "rk_npu_f32i8f32_run_static": (C.c_int, [_P, _P, _P, _P, _P]),
    "rk_npu_b200_matmul_launch_count": (C.c_uint64, [_P]),
    "rk_npu_w4a8_family_config_init": (None, [C.POINTER(W4A8FamilyConfig), C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]),
    # search tuner
    "rk_npu_w4a8_autotune": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, _P, C.POINTER(W4A8Strategy), C.POINTER(W4A8Strategy)]),
    "rk_npu_w4a8_autotune_ex": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, _P, C.POINTER(W4A8StrategyEx),
                                          C.POINTER(W4A8StrategyEx)]),
    "rk_npu_w4a8_autotune_cached": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, _P, C.c_char_p, C.c_int,
                                              C.POINTER(W4A8Strategy), C.POINTER(W4A8Strategy), C.POINTER(C.c_int)]),
    "rk_npu_w4a8_autotune_cached_ex": (C.c_int, [_P, C.POINTER(W4A8AutotuneConfig), _P, _P, C.c_char_p, C.c_int,
                                                 C.POINTER(W4A8StrategyEx), C.POINTER(W4A8StrategyEx), C.POINTER(C.c_int)]),
    "rk_npu_w4a8_autotune_family": (C.c_int, [_P, C.POINTER(W4A8FamilyConfig), _P, _P, C.POINTER(W4A8FamilySummary),
                                              C.POINTER(W4A8Strategy), C.POINTER(W4A8FamilySummary), C.POINTER(W4A8Strategy)]),
    "rk_npu_w4a8_autotune_family_ex": (C.c_int, [_P, C.POINTER(W4A8FamilyConfig), _P, _P, C.POINTER(W4A8FamilySummary),
                                                 C.POINTER(W4A8StrategyEx), C.POINTER(W4A8FamilySummary),
                                                 C.POINTER(W4A8StrategyEx)]),
    "rk_npu_w4a8_autotune_family_cached": (C.c_int, [_P, C.POINTER(W4A8FamilyConfig), _P, _P, C.c_char_p, C.c_int,
                                                     C.POINTER(W4A8FamilySummary), C.POINTER(W4A8Strategy),
                                                     C.POINTER(W4A8FamilySummary), C.POINTER(W4A8Strategy),
                                                     C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "rk_npu_w4a8_autotune_family_cached_ex": (C.c_int, [_P, C.POINTER(W4A8FamilyConfig), _P, _P, C.c_char_p, C.c_int,
                                                        C.POINTER(W4A8FamilySummary), C.POINTER(W4A8StrategyEx),
                                                        C.POINTER(W4A8FamilySummary), C.POINTER(W4A8StrategyEx),
                                                        C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    # B200 extensions
    "rk_npu_b200_device": (C.c_int, [_P]),
    "rk_npu_b200_driver_version": (C.c_uint32, [_P]),
    "rk_npu_b200_group_id": (C.c_int, [_P]),
    "rk_npu_b200_open_group": (_P, [C.c_char_p, C.c_int, C.c_int, _P]),
    "rk_npu_b200_group_rank": (C.c_int, [_P]),
    "rk_npu_b200_group_size": (C.c_int, [_P]),
    "rk_npu_b200_shard_columns": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "rk_npu_b200_w4a8_workspace_shard": (C.c_int, [_P, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "rk_npu_b200_w4a8_enqueue_local_f16": (C.c_int, [_P, _P, _P, _P, _P]),
    "rk_npu_b200_w4a8_enqueue_local_f32": (C.c_int, [_P, _P, _P, _P, _P]),
    "rk_npu_b200_group_all_gather": (C.c_int, [_P, _P, C.c_size_t, _P]),
    "rk_npu_b200_w4a8_enqueue_batch_f16": (C.c_int, [C.c_int, C.POINTER(_P), C.POINTER(_P), C.POINTER(_P), C.POINTER(_P), _P]),
    "rk_npu_b200_open_offline": (_P, [C.c_uint32]),
    "rk_npu_b200_w4a8_enqueue_f32": (C.c_int, [_P, _P, _P, _P, _P]),
    "rk_npu_b200_w4a8_enqueue_f16": (C.c_int, [_P, _P, _P, _P, _P]),
    # routed experts (include/rknpu_b200_moe.h)
    "rk_npu_moe_w8_config_init": (None, [C.POINTER(MoeConfig), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "rk_npu_moe_w8_weights_create": (_P, [_P, C.POINTER(MoeWeightConfig), C.POINTER(MoeExpert)]),
    "rk_npu_moe_w8_weights_free": (None, [_P]),
    "rk_npu_moe_w8_workspace_create": (_P, [_P, C.POINTER(MoeConfig)]),
    "rk_npu_moe_w8_workspace_free": (None, [_P]),
    "rk_npu_moe_w8_weights_device_bytes": (C.c_uint64, [_P]),
    "rk_npu_moe_w8_workspace_device_bytes": (C.c_uint64, [_P]),
    "rk_npu_moe_w8_run_quantized": (C.c_int, [_P, _P, C.c_int, _P, _P, _P, _P, _P, C.POINTER(MoeTimings)]),
    "rk_npu_moe_w8_run_f32": (C.c_int, [_P, _P, C.c_int, _P, _P, _P, _P, C.POINTER(MoeTimings)]),
    "rk_npu_moe_quant_weights_create": (_P, [_P, C.POINTER(MoeWeightConfig), C.POINTER(MoeExpert)]),
    "rk_npu_moe_quant_weights_create_full_k": (_P, [_P, C.POINTER(MoeWeightConfig), C.POINTER(MoeExpert)]),
    "rk_npu_moe_quant_workspace_create": (_P, [_P, C.POINTER(MoeConfig)]),
    "rk_npu_moe_w4_weights_create": (_P, [_P, C.POINTER(MoeWeightConfig), C.POINTER(MoeExpert)]),
    "rk_npu_moe_w4_workspace_create": (_P, [_P, C.POINTER(MoeConfig)]),
    "rk_npu_moe_w4_slots_create": (_P, [_P, C.POINTER(MoeWeightConfig), C.POINTER(MoeExpert)]),
    "rk_npu_moe_quant_slots_create": (_P, [_P, C.POINTER(MoeWeightConfig)]),
    "rk_npu_moe_quant_expert_blob_bytes": (C.c_uint64, [_P]),
    "rk_npu_moe_quant_export_expert": (C.c_int, [_P, C.c_int, _P, C.c_uint64]),
    "rk_npu_moe_quant_import_expert": (C.c_int, [_P, C.c_int, _P, C.c_uint64]),
    "rk_npu_moe_quant_import_expert_timed": (C.c_int, [_P, C.c_int, _P, C.c_uint64, C.POINTER(MoeImportTimings)]),
    "rk_npu_moe_quant_swap_slots": (C.c_int, [_P, C.c_int, _P, C.c_int]),
    "rk_npu_b200_w4a8_enqueue_swiglu_f32": (C.c_int, [_P, _P, _P, _P, _P]),
    "rk_npu_b200_w4a8_enqueue_ffn_f32": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P]),
    "rk_npu_b200_w4a8_enqueue_swiglu_collect_f32": (C.c_int, [_P, _P, _P, _P, _P, _P]),
    "rk_npu_b200_w4a8_enqueue_quantize_slice": (C.c_int, [_P, _P, _P, _P, _P]),
    "rk_npu_b200_w4a8_enqueue_codes_f32": (C.c_int, [_P, _P, _P, C.c_int, _P, _P, _P]),
    "rk_npu_b200_w4a8_finish": (C.c_int, [_P]),
    "rk_npu_b200_w4a8_run_acc_i32": (C.c_int, [_P, _P, _P, C.c_int, _P]),
    "rk_npu_b200_w4a8_last_quant": (C.c_int, [_P, _P, _P]),
    "rk_npu_b200_w4a8_set_schedule": (C.c_int, [_P, C.c_int, C.c_int]),
    "rk_npu_b200_w4a8_schedule": (C.c_int, [_P, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "rk_npu_b200_w4a8_enqueue_f16_static": (C.c_int, [_P, _P, _P, C.c_int, _P]),
    "rk_npu_b200_w4a8_static_status": (C.c_int, [_P, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "rk_npu_mem_alloc": (C.c_int, [_P, C.c_uint64, C.c_uint32, C.POINTER(Mem)]),
    "rk_npu_mem_view": (C.c_int, [C.POINTER(Mem), C.c_uint64, C.c_uint64, C.POINTER(Mem)]),
    "rk_npu_mem_sync": (C.c_int, [_P, C.POINTER(Mem), C.c_int]),
    "rk_npu_mem_free": (C.c_int, [_P, C.POINTER(Mem)]),
    "rk_npu_mem_import_dmabuf": (C.c_int, [_P, C.c_int, _P, C.c_uint64, C.c_uint32, C.POINTER(Mem)]),
    "rk_npu_mem_export_dmabuf": (C.c_int, [_P, C.POINTER(Mem), C.POINTER(C.c_int)]),
    "rk_npu_add_rmsnorm_f16_config_init": (None, [C.POINTER(AddRmsNormConfig), C.c_int, C.c_int]),
    "rk_npu_add_rmsnorm_f16_query": (C.c_int, [C.POINTER(AddRmsNormConfig), C.POINTER(AddRmsNormSizes)]),
    "rk_npu_add_rmsnorm_f16_plan_create": (_P, [_P, C.POINTER(AddRmsNormConfig), _P]),
    "rk_npu_add_rmsnorm_f16_run": (C.c_int, [_P, _P, C.POINTER(Mem), C.POINTER(Mem), C.POINTER(Mem), C.POINTER(Mem)]),
    "rk_npu_add_rmsnorm_f16_plan_free": (None, [_P]),
    "rk_npu_b200_add_rmsnorm_f16_enqueue": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, _P, _P]),
    "rk_npu_b200_test_fail_allocation": (None, [C.c_longlong]),
    "rk_npu_b200_w4a8_test_starve": (C.c_int, [_P, C.c_int]),
    "rk_npu_b200_w4a8_test_device_error": (C.c_int, [_P]),
    "rk_npu_b200_w4a8_launch_count": (C.c_uint64, [_P]),
    "rk_npu_b200_w4a8_trace_enable": (C.c_int, [_P, C.c_int]),
    "rk_npu_b200_w4a8_trace_read": (C.c_int, [_P, _P, C.c_int]),
}

_lib = None


def declared_symbols():
    """Names of every entry point the headers declare."""
    return sorted(_SIGNATURES)


def load() -> C.CDLL:
    """Load the built library and attach the prototypes. Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is not built: run `python -c 'import __graft_entry__ as g; g.build()'` "
                           "(nvcc, sm_100a). There is no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
