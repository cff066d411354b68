"""Mutable slot banks of int4 experts and their cache records (include/rk_npu_moe_w8.h:113-146) through the C ABI.

What is checked follows the original's board test of this interface (tests/test_moe_quant.cpp:236-356, :84-180): a
record exported from an immutable bank, imported into another physical slot and exported again is the same bytes; a
run through any slot permutation equals the run on the resident experts bit for bit; records of the all-int4, the
whole-K certified and the mixed (int4 routed + int8 shared) forms are interchangeable; a staging bank is filled by
another thread while the hot bank computes, slots are promoted by exchange, and the hot bank survives the staging
bank's destruction; short, untagged, foreign and non-positive-scale records are refused and leave the slot as it was.
That test also counts the original's internal buffer synchronisations through linker wraps, which has no meaning
here; the rest is restated, not compiled."""
import ctypes as C
import threading

import numpy as np
import pytest

import rknpu2_matmul_open_b200 as rk
from conftest import bits
from rknpu2_matmul_open_b200 import capi, moe

pytestmark = pytest.mark.gpu


def int4_experts(H, I, E, seed, small_first=False):
    rng = np.random.default_rng(seed)
    ex = dict(gate_up=rng.integers(-7, 8, size=(E, H, 2 * I), dtype=np.int8),
              gate_up_scales=(1e-3 * (1 + np.arange(2 * I) % 13)).astype(np.float32)[None].repeat(E, 0),
              down=rng.integers(-7, 8, size=(E, I, H), dtype=np.int8),
              down_scales=(1e-3 * (1 + np.arange(H) % 7)).astype(np.float32)[None].repeat(E, 0))
    if small_first:
        ex["gate_up"][0] //= 4          # expert 0 also certifies the whole of K (tests/test_moe_quant.cpp:193-194)
    return ex


def record_part(K, N):
    """Bytes of one [K, N] int4 matrix in a record: K padded to a multiple of 128, two codes per byte."""
    return -(-K // 128) * 128 * N // 2


def rows_of(n, H):
    return (np.sin((np.arange(n * H) % 97) * 0.13) * 0.3).astype(np.float32).reshape(n, H)


def run(ws, w, x, ids, routes):
    out = np.full(x.shape, np.float32(7), np.float32)
    assert ws.run_f32(w, x, np.ascontiguousarray(ids, np.int32), np.ascontiguousarray(routes, np.float32), out) == capi.RK_NPU_OK
    return out


@pytest.mark.parametrize("H,I,E", [(2048, 512, 3), (256, 64, 5), (576, 128, 4)])
def test_records_round_trip_and_slots_compute_like_resident_experts(gpu, H, I, E):
    _, dom, _ = gpu
    ex = int4_experts(H, I, E, seed=H + E)
    resident = moe.MoeWeights(dom, form="quant", **ex)
    work = moe.MoeWorkspace(dom, moe.default_config(H, I, E, 0, 2, 16), form="quant")
    bank = moe.MoeWeights.slot_bank(dom, H, I, E)
    bank_work = moe.MoeWorkspace(dom, moe.default_config(H, I, E, 0, 1, 16), form="quant")
    need = resident.record_bytes()
    assert need == bank.record_bytes() == record_part(H, 2 * I) + record_part(I, H) + 4 * (2 * I + H) + 16      # + scales + trailer
    assert bank.device_bytes() == E * (need - 16)
    stride = (need + 4095) // 4096 * 4096                    # a file store may page-align its records
    record, again = np.zeros(stride, np.uint8), np.ones(stride, np.uint8)
    x = rows_of(5, H)
    # an empty slot contributes zero
    assert not run(bank_work, bank, x, np.zeros((5, 1)), np.ones((5, 1))).any()
    for expert in (0, E - 1, 1, 0):
        physical = (expert + 1) % E
        assert resident.export_expert(expert, record) == capi.RK_NPU_OK
        assert bank.import_expert(physical, record) == capi.RK_NPU_OK
        assert bank.export_expert(physical, again) == capi.RK_NPU_OK
        assert np.array_equal(record[:need], again[:need])
        want = run(work, resident, x, np.full((5, 2), expert), np.tile([1.0, 0.0], (5, 1)))
        got = run(bank_work, bank, x, np.full((5, 1), physical), np.ones((5, 1)))
        assert np.array_equal(bits(got), bits(want))
    for expert in range(E):                                   # every slot filled: a permutation of all experts
        assert resident.export_expert(expert, record) == capi.RK_NPU_OK and bank.import_expert((expert + 1) % E, record) == capi.RK_NPU_OK
    ids = (np.arange(5) % E)[:, None]
    want = run(work, resident, x, np.concatenate([ids, ids], 1), np.tile([1.0, 0.0], (5, 1)))
    assert np.array_equal(bits(run(bank_work, bank, x, (ids + 1) % E, np.ones((5, 1)))), bits(want))

    # refusals: nothing is copied, the slot keeps its expert
    assert resident.export_expert(0, record) == capi.RK_NPU_OK
    keep = np.zeros(need, np.uint8)
    assert bank.export_expert(0, keep) == capi.RK_NPU_OK
    assert bank.import_expert(0, record, nbytes=need - 1) == capi.RK_NPU_ERR_PARAM                    # short
    assert bank.export_expert(0, again[:need - 1]) == capi.RK_NPU_ERR_PARAM
    for slot in (-1, E):
        assert bank.import_expert(slot, record) == capi.RK_NPU_ERR_PARAM and bank.export_expert(slot, again) == capi.RK_NPU_ERR_PARAM
    bad = record.copy()
    bad[need - 4:need].view(np.int32)[0] &= ~7                                                       # untagged (tests/test_moe_quant.cpp:347-353)
    assert bank.import_expert(0, bad) == capi.RK_NPU_ERR_PARAM
    bad = record.copy()
    bad[need - 4:need].view(np.int32)[0] = 2 if not 512 < H <= 2048 else 3                           # whole-K tag where it cannot hold / unknown tag
    assert bank.import_expert(0, bad) == capi.RK_NPU_ERR_PARAM
    bad = record.copy()
    bad[need - 16:need - 12] = 0                                                                      # not one of this library's records
    assert bank.import_expert(0, bad) == capi.RK_NPU_ERR_PARAM
    bad = record.copy()
    bad[need - 12:need - 8].view(np.int32)[0] = H + 64                                                # another geometry
    assert bank.import_expert(0, bad) == capi.RK_NPU_ERR_PARAM
    scales_at = record_part(H, 2 * I) + record_part(I, H)
    for value in (0.0, -1.0, np.inf, np.nan):
        bad = record.copy()
        bad[scales_at + 4 * 3:scales_at + 4 * 4].view(np.float32)[0] = value
        assert bank.import_expert(0, bad) == capi.RK_NPU_ERR_PARAM
    assert bank.lib.rk_npu_moe_quant_import_expert(bank.handle, 0, None, need) == capi.RK_NPU_ERR_PARAM
    assert bank.lib.rk_npu_moe_quant_import_expert(None, 0, record.ctypes.data, need) == capi.RK_NPU_ERR_PARAM
    assert bank.export_expert(0, again) == capi.RK_NPU_OK and np.array_equal(again[:need], keep)
    # an int8 bank has no records
    w8 = moe.MoeWeights(dom, **ex)
    assert w8.record_bytes() == 0 and w8.export_expert(0, again) == capi.RK_NPU_ERR_PARAM and w8.import_expert(0, record) == capi.RK_NPU_ERR_PARAM
    for h in (w8, bank_work, bank, work, resident):
        h.free()


def test_staged_import_exchange_and_survival(gpu):
    _, dom, _ = gpu
    H, I, E, rows = 1024, 256, 3, 5
    ex = int4_experts(H, I, E, seed=11, small_first=True)
    resident = moe.MoeWeights(dom, form="quant_full_k", **ex)
    work = moe.MoeWorkspace(dom, moe.default_config(H, I, E, 0, 2, 8), form="quant")
    hot, stage = moe.MoeWeights.slot_bank(dom, H, I, E), moe.MoeWeights.slot_bank(dom, H, I, E)
    one = moe.MoeWorkspace(dom, moe.default_config(H, I, E, 0, 1, 8), form="quant")
    need = resident.record_bytes()
    bank_bytes = hot.device_bytes()
    assert bank_bytes and stage.device_bytes() == bank_bytes
    records = [np.zeros(need, np.uint8) for _ in range(E)]
    for e in range(E):
        assert resident.export_expert(e, records[e]) == capi.RK_NPU_OK and hot.import_expert(e, records[e]) == capi.RK_NPU_OK
    x = rows_of(rows, H)
    physical = (np.arange(rows) % E)[:, None]
    want = None
    for iteration in range(5):
        failures = []

        def importer():
            for slot in range(E):
                t = capi.MoeImportTimings()
                if stage.import_expert(slot, records[(iteration + slot) % E], t) != capi.RK_NPU_OK:
                    failures.append(("rc", slot))
                if not (t.validate_us >= 0 and t.gate_sync_us > 0 and t.down_sync_us >= 0 and t.total_us >= t.gate_sync_us):
                    failures.append(("timings", slot))

        thread = threading.Thread(target=importer)
        thread.start()
        run(one, hot, x, physical, np.ones((rows, 1)))          # the hot bank computes while the staging bank is filled
        thread.join()
        assert not failures
        for slot in range(E):
            assert hot.swap_slot(slot, stage, slot) == capi.RK_NPU_OK
            assert hot.device_bytes() == bank_bytes and stage.device_bytes() == bank_bytes
        source = ((iteration + np.arange(rows) % E) % E)[:, None]
        want = run(work, resident, x, np.concatenate([source, source], 1), np.tile([1.0, 0.0], (rows, 1)))
        assert np.array_equal(bits(run(one, hot, x, physical, np.ones((rows, 1)))), bits(want))

    # exchanges of slot 0 beside imports into slot 1 of the same staging bank
    done = threading.Event()
    failures = []

    def importer():
        for _ in range(200):
            if stage.record_bytes() != need or stage.import_expert(1, records[0]) != capi.RK_NPU_OK:
                failures.append("import")
        done.set()

    thread = threading.Thread(target=importer)
    thread.start()
    swaps = 0
    while not done.is_set() or swaps == 0:
        assert hot.swap_slot(0, stage, 0) == capi.RK_NPU_OK
        swaps += 1
    thread.join()
    assert not failures and swaps > 0
    if swaps % 2:
        assert hot.swap_slot(0, stage, 0) == capi.RK_NPU_OK
    out = np.zeros(need, np.uint8)
    assert stage.export_expert(1, out) == capi.RK_NPU_OK and np.array_equal(out, records[0])
    before = dom.memory_stats().live_bytes
    stage.free()
    assert dom.memory_stats().live_bytes == before - bank_bytes       # the staging bank took its own slots with it, and only those
    assert hot.device_bytes() == bank_bytes
    assert np.array_equal(bits(run(one, hot, x, physical, np.ones((rows, 1)))), bits(want))

    # exchange: all-int4 slot banks of one geometry, context and domain only
    other = moe.MoeWeights.slot_bank(dom, H, 2 * I, E)
    assert hot.swap_slot(0, other, 0) == capi.RK_NPU_ERR_PARAM
    assert hot.swap_slot(0, resident, 0) == capi.RK_NPU_ERR_PARAM        # an immutable bank is one allocation here
    assert hot.swap_slot(E, hot, 0) == capi.RK_NPU_ERR_PARAM and hot.swap_slot(0, hot, -1) == capi.RK_NPU_ERR_PARAM
    assert hot.lib.rk_npu_moe_quant_swap_slots(hot.handle, 0, None, 0) == capi.RK_NPU_ERR_PARAM
    far = moe.MoeWeights.slot_bank(gpu[2], H, I, E)
    assert hot.swap_slot(0, far, 0) == capi.RK_NPU_ERR_PARAM             # another domain
    assert hot.swap_slot(0, hot, 1) == capi.RK_NPU_OK and hot.swap_slot(0, hot, 1) == capi.RK_NPU_OK
    for h in (far, other, one, hot, work, resident):
        h.free()


def test_mixed_slots_with_a_shared_int8_expert(gpu, oracle):
    _, dom, _ = gpu
    H, I, E, K = 1024, 128, 3, 2
    ex = int4_experts(H, I, E, seed=23, small_first=True)
    ex["gate_up"][1:, :, 0] = 7            # a column that overflows an INT16 partial over K = 1024 but fits two slices of 512
    rng = np.random.default_rng(5)
    shared = (rng.integers(-127, 128, size=(H, 2 * I), dtype=np.int8), np.full(2 * I, 3e-4, np.float32),
              rng.integers(-127, 128, size=(I, H), dtype=np.int8), np.full(H, 4e-4, np.float32))
    all_ex = {k: np.concatenate([ex[k], shared[i][None]], 0) for i, k in enumerate(("gate_up", "gate_up_scales", "down", "down_scales"))}
    packed = moe.MoeWeights(dom, form="quant_full_k", **ex)
    mixed = moe.MoeWeights(dom, shared_expert=1, form="w4", **all_ex)
    slots = moe.MoeWeights.slot_bank(dom, H, I, E, shared=shared)
    need = packed.record_bytes()
    assert slots.record_bytes() == need == mixed.record_bytes()
    lib = capi.load()
    cfg0, cfg1 = capi.MoeWeightConfig(H, I, E, 0), capi.MoeWeightConfig(H, I, E, 1)
    expert = capi.MoeExpert(*(a.ctypes.data for a in shared))
    assert lib.rk_npu_moe_w4_slots_create(dom.handle, C.byref(cfg0), C.byref(expert)) is None       # needs shared_expert = 1
    assert lib.rk_npu_moe_w4_slots_create(dom.handle, C.byref(cfg1), None) is None                  # and the shared weights
    assert lib.rk_npu_moe_quant_slots_create(dom.handle, C.byref(cfg1)) is None                     # the all-int4 bank has no shared expert
    assert lib.rk_npu_moe_quant_slots_create(None, C.byref(cfg0)) is None
    record, again = np.zeros(need, np.uint8), np.zeros(need, np.uint8)
    assert slots.import_expert(E, record) == capi.RK_NPU_ERR_PARAM and slots.export_expert(E, record) == capi.RK_NPU_ERR_PARAM   # the shared expert is no record
    assert mixed.export_expert(E, record) == capi.RK_NPU_ERR_PARAM
    work = moe.MoeWorkspace(dom, moe.default_config(H, I, E, 1, K, 128), form="w4")
    tags = set()
    for rotation, rows in enumerate((1, 5, 128, 1)):
        for e in range(E):
            slot = (e + rotation) % E
            assert packed.export_expert(e, record) == capi.RK_NPU_OK and mixed.export_expert(e, again) == capi.RK_NPU_OK
            assert np.array_equal(record, again)               # the whole-K certified and the mixed form pack alike
            tags.add(int(record[need - 4:need].view(np.int32)[0]))
            assert slots.import_expert(slot, record) == capi.RK_NPU_OK
            assert slots.export_expert(slot, again) == capi.RK_NPU_OK and np.array_equal(record, again)
        r = np.arange(rows)[:, None]
        k = np.arange(K)[None]
        ids = (r + np.where(r % 2 == 1, k, 0)) % E             # duplicate routes; sums that are not 1; rows without routed experts
        routes = np.where((r % 3 == 2) | ((r % 3 == 1) & (k > 0)), 0.0, np.where(k > 0, 0.375, 0.875))
        x = rows_of(rows, H)
        want = run(work, mixed, x, ids, routes)
        got = run(work, slots, x, (ids + rotation) % E, routes)
        assert np.array_equal(bits(got), bits(want))
        if rows > 2:
            assert got[2].any()                                # the shared expert alone (coefficient 1)
        _, q, s = oracle.moe_quantize_rows(x)
        rc, ref = oracle.moe_run(all_ex, 1, K, q, s, ids.astype(np.int32), routes.astype(np.float32), mode=1)
        assert rc == 0 and np.array_equal(bits(got), bits(ref))
    assert tags == {1, 2}                                      # expert 0 certifies the whole of K, the others only slices
    # a record of another geometry's bank is refused by the trailer, a record of the plain all-int4 form is accepted
    plain = moe.MoeWeights(dom, form="quant", **ex)
    assert plain.export_expert(1, record) == capi.RK_NPU_OK and int(record[need - 4:need].view(np.int32)[0]) == 1
    assert slots.import_expert(1, record) == capi.RK_NPU_OK
    for h in (plain, work, slots, mixed, packed):
        h.free()
