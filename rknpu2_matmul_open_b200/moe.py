"""Host-side mirror of the routed-experts operator (include/rknpu_b200_moe.h) over the C ABI.

``MoeWeights`` wraps rk_npu_moe_w8_weights (int8 experts, copied and packed at creation), ``MoeWorkspace`` wraps
rk_npu_moe_w8_workspace; the run methods have the argument meaning and return codes of the C calls (host arrays
in, host array out, blocking).  All compute happens in the CUDA library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .capi import MoeConfig, MoeExpert, MoeImportTimings, MoeTimings, MoeWeightConfig
from .w4a8 import W4A8Error, _ptr


def default_config(hidden: int, intermediate: int, routed_experts: int, shared_expert: int, top_k: int, max_rows: int) -> MoeConfig:
    """rk_npu_moe_w8_config_init"""
    c = MoeConfig()
    capi.load().rk_npu_moe_w8_config_init(C.byref(c), hidden, intermediate, routed_experts, shared_expert, top_k, max_rows)
    return c


class MoeWeights:
    """rk_npu_moe_w8_weights_create / _free.  gate_up [E, H, 2I] int8, gate_up_scales [E, 2I], down [E, I, H] int8,
    down_scales [E, H]; E = routed + shared experts, the shared one last."""

    def __init__(self, domain, gate_up, gate_up_scales, down, down_scales, shared_expert: int = 0, form: str = "w8"):
        """form: 'w8' int8 experts; 'quant' / 'quant_full_k' all experts int4 codes; 'w4' routed int4 + shared int8."""
        self.lib = capi.load()
        gate_up = np.ascontiguousarray(gate_up, np.int8)
        down = np.ascontiguousarray(down, np.int8)
        gus = np.ascontiguousarray(gate_up_scales, np.float32)
        dns = np.ascontiguousarray(down_scales, np.float32)
        E, H, I2 = gate_up.shape
        self.config = MoeWeightConfig(H, I2 // 2, E - shared_expert, shared_expert)
        experts = (MoeExpert * E)()
        for e in range(E):
            experts[e] = MoeExpert(_ptr(gate_up[e]), _ptr(gus[e]), _ptr(down[e]), _ptr(dns[e]))
        name = {"w8": "rk_npu_moe_w8_weights_create", "quant": "rk_npu_moe_quant_weights_create",
                "quant_full_k": "rk_npu_moe_quant_weights_create_full_k", "w4": "rk_npu_moe_w4_weights_create"}[form]
        self.handle = getattr(self.lib, name)(domain.handle, C.byref(self.config), experts)
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_PARAM, name)

    @classmethod
    def slot_bank(cls, domain, hidden: int, intermediate: int, routed_experts: int, shared=None) -> "MoeWeights":
        """rk_npu_moe_quant_slots_create (shared is None: every slot an int4 expert) or rk_npu_moe_w4_slots_create
        (shared = (gate_up [H, 2I] int8, gate_up_scales, down [I, H] int8, down_scales): the immutable int8 shared expert).
        Slots hold nothing until records are imported."""
        self = cls.__new__(cls)
        self.lib = capi.load()
        self.config = MoeWeightConfig(hidden, intermediate, routed_experts, 0 if shared is None else 1)
        if shared is None:
            name = "rk_npu_moe_quant_slots_create"
            self.handle = self.lib.rk_npu_moe_quant_slots_create(domain.handle, C.byref(self.config))
        else:
            name = "rk_npu_moe_w4_slots_create"
            gu, gus, dn, dns = (np.ascontiguousarray(a, t) for a, t in zip(shared, (np.int8, np.float32, np.int8, np.float32)))
            expert = MoeExpert(_ptr(gu), _ptr(gus), _ptr(dn), _ptr(dns))
            self.handle = self.lib.rk_npu_moe_w4_slots_create(domain.handle, C.byref(self.config), C.byref(expert))
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_PARAM, name)
        return self

    def device_bytes(self) -> int:
        return int(self.lib.rk_npu_moe_w8_weights_device_bytes(self.handle))

    def record_bytes(self) -> int:
        """rk_npu_moe_quant_expert_blob_bytes: the size of one int4 expert's cache record (0: the bank has none)."""
        return int(self.lib.rk_npu_moe_quant_expert_blob_bytes(self.handle))

    def export_expert(self, expert: int, out: np.ndarray) -> int:
        """rk_npu_moe_quant_export_expert into a uint8 array; returns the C return code."""
        return self.lib.rk_npu_moe_quant_export_expert(self.handle, expert, _ptr(out), out.nbytes)

    def import_expert(self, slot: int, record: np.ndarray, timings: MoeImportTimings | None = None, nbytes: int | None = None) -> int:
        """rk_npu_moe_quant_import_expert[_timed] from a uint8 array; returns the C return code."""
        size = record.nbytes if nbytes is None else nbytes
        if timings is None:
            return self.lib.rk_npu_moe_quant_import_expert(self.handle, slot, _ptr(record), size)
        return self.lib.rk_npu_moe_quant_import_expert_timed(self.handle, slot, _ptr(record), size, C.byref(timings))

    def swap_slot(self, slot: int, other: "MoeWeights", other_slot: int) -> int:
        """rk_npu_moe_quant_swap_slots; returns the C return code."""
        return self.lib.rk_npu_moe_quant_swap_slots(self.handle, slot, other.handle, other_slot)

    def free(self):
        if self.handle:
            self.lib.rk_npu_moe_w8_weights_free(self.handle)
            self.handle = None


class MoeWorkspace:
    """rk_npu_moe_w8_workspace_create / _free and the two run calls."""

    def __init__(self, domain, config: MoeConfig, form: str = "w8"):
        self.lib = capi.load()
        self.config = config
        name = {"w8": "rk_npu_moe_w8_workspace_create", "quant": "rk_npu_moe_quant_workspace_create",
                "quant_full_k": "rk_npu_moe_quant_workspace_create", "w4": "rk_npu_moe_w4_workspace_create"}[form]
        self.handle = getattr(self.lib, name)(domain.handle, C.byref(config))
        if not self.handle:
            raise W4A8Error(capi.RK_NPU_ERR_PARAM, name)

    def device_bytes(self) -> int:
        return int(self.lib.rk_npu_moe_w8_workspace_device_bytes(self.handle))

    def run_quantized(self, weights: MoeWeights, codes, row_scales, expert_ids, route_weights, out, timings: MoeTimings | None = None) -> int:
        return self.lib.rk_npu_moe_w8_run_quantized(self.handle, weights.handle, int(codes.shape[0]), _ptr(codes), _ptr(row_scales),
                                                    _ptr(expert_ids), _ptr(route_weights), _ptr(out),
                                                    C.byref(timings) if timings is not None else None)

    def run_f32(self, weights: MoeWeights, rows, expert_ids, route_weights, out, timings: MoeTimings | None = None) -> int:
        return self.lib.rk_npu_moe_w8_run_f32(self.handle, weights.handle, int(rows.shape[0]), _ptr(rows), _ptr(expert_ids),
                                              _ptr(route_weights), _ptr(out), C.byref(timings) if timings is not None else None)

    def free(self):
        if self.handle:
            self.lib.rk_npu_moe_w8_workspace_free(self.handle)
            self.handle = None
