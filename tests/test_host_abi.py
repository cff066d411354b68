"""Host logic behind the C ABI that needs no GPU: the library loads and exports every
declared entry point, the accounting and validation arithmetic equals the reference's,
and tuning-cache files round-trip and interoperate with the reference's own build."""
import ctypes as C
import os
import re
from pathlib import Path

import numpy as np
import pytest

from rknpu2_matmul_open_b200 import capi
from rknpu2_matmul_open_b200.capi import (I4WeightConfig, W4A8AutotuneConfig, W4A8Config, W4A8MemoryInfo,
                                          W4A8MemoryInfoEx, W4A8Options, W4A8Strategy, W4A8StrategyEx)

ROOT = Path(__file__).resolve().parents[1]


def cfg_of(lib, m, n, k, **kw):
    c = W4A8Config()
    lib.rk_npu_w4a8_config_init(C.byref(c), m, n, k)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def test_library_exports_every_declared_symbol(lib):
    declared = set()
    for header in ("rknpu_b200_w4a8.h", "rknpu_b200_quant.h", "rknpu_b200_moe.h", "rknpu_b200_rmsnorm.h", "rknpu_b200_ext.h"):
        text = (ROOT / "include" / header).read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        declared |= set(re.findall(r"\b(rk_npu_\w+)\s*\(", text))
    assert declared == set(capi.declared_symbols()), declared ^ set(capi.declared_symbols())
    for name in declared:
        assert hasattr(lib, name), name


def _abi_layout():
    import importlib.util
    spec = importlib.util.spec_from_file_location("abi_layout", ROOT / "tests" / "golden" / "abi_layout.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_struct_layouts_and_constants_equal_the_original_headers():
    # tests/golden/reference_abi_layout.txt holds, for every struct, member, enumerator and macro constant that
    # include/*.h declares, the size / offset / value a C compiler derives from the ORIGINAL project's headers; the same
    # program compiled against include/*.h must print the same text, so a caller compiled against either header
    # passes structs this library reads correctly.
    abi = _abi_layout()
    structs, constants = abi.declared_names()
    assert len(structs) == 32 and "rk_npu_moe_w8_timings" in structs and "RK_NPU_ERR_BUSY" in constants
    assert structs["rk_npu_moe_w8_timings"][:3] == ["input_us", "schedule_us", "build_us"]      # "double a, b, c;"
    ours = abi.layout(ROOT / "include", abi.OURS)
    golden = (ROOT / "tests" / "golden" / "reference_abi_layout.txt").read_text()
    assert ours == golden
    default = re.search(r"^REF\s*\?=\s*(\S+)", (ROOT / "oracle" / "Makefile").read_text(), flags=re.M).group(1)
    reference = Path(os.environ.get("REF", default)) / "include"      # where oracle/Makefile looks for the original tree
    if reference.is_dir():           # where the original tree is at hand, the golden file itself is re-derived
        assert abi.layout(reference, abi.THEIRS) == golden
        assert abi.functions(reference, abi.THEIRS) == (ROOT / "tests" / "golden" / "reference_header_symbols.txt").read_text().split()


def test_ctypes_mirrors_have_the_c_sizes():
    # the Python structs the tests and the bench pass through the ABI are the sizes the C headers give
    abi = _abi_layout()
    text = abi.layout(ROOT / "include", abi.OURS).splitlines()
    sizes = dict(line.split()[1:3] for line in text if line.startswith("sizeof"))
    offsets = {tuple(line.split()[1:3]): int(line.split()[3]) for line in text if line.startswith("offsetof")}
    mirrors = {"rk_npu_w4a8_config": capi.W4A8Config, "rk_npu_w4a8_options": capi.W4A8Options,
               "rk_npu_w4a8_memory_info": capi.W4A8MemoryInfo, "rk_npu_w4a8_memory_info_ex": capi.W4A8MemoryInfoEx,
               "rk_npu_w4a8_strategy": capi.W4A8Strategy, "rk_npu_w4a8_strategy_ex": capi.W4A8StrategyEx,
               "rk_npu_w4a8_autotune_config": capi.W4A8AutotuneConfig, "rk_npu_i4_weight_config": capi.I4WeightConfig,
               "rk_npu_moe_w8_weight_config": capi.MoeWeightConfig, "rk_npu_moe_w8_config": capi.MoeConfig,
               "rk_npu_moe_w8_expert": capi.MoeExpert, "rk_npu_moe_w8_timings": capi.MoeTimings, "rk_npu_mem": capi.Mem,
               "rk_npu_add_rmsnorm_f16_config": capi.AddRmsNormConfig, "rk_npu_add_rmsnorm_f16_sizes": capi.AddRmsNormSizes,
               "rk_npu_domain_memory_stats": capi.DomainMemoryStats}
    for name, mirror in mirrors.items():
        assert C.sizeof(mirror) == int(sizes[name]), name
        for field, _ in mirror._fields_:
            assert getattr(mirror, field).offset == offsets[(name, field)], (name, field)


def test_no_gpu_means_open_fails_loudly(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert not lib.rk_npu_open(None)          # no CPU fallback: without a device there is no context
    assert not lib.rk_npu_open(b"cuda:0")
    assert not lib.rk_npu_open(b"renderD128")


def test_defaults_and_strerror(lib):
    c = cfg_of(lib, 7, 65, 513)
    assert (c.M, c.N, c.K, c.m_tile, c.k_tile, c.n_tile, c.npu_core_mask, c.timeout_ms, c.pipeline, c.cpu_threads) == \
        (7, 65, 513, 64, 480, 1024, 1, 500, 1, 1)
    o = W4A8Options()
    lib.rk_npu_w4a8_options_init(C.byref(o))
    assert (o.struct_size, o.input_layout, o.reduce_backend) == (C.sizeof(W4A8Options), 0, 0)
    a = W4A8AutotuneConfig()
    lib.rk_npu_w4a8_autotune_config_init(C.byref(a), 1, 2, 3)
    assert (a.M, a.N, a.K, a.activation_type, a.allowed_npu_core_mask, a.allowed_cpu_core_mask, a.warmup, a.loops,
            a.repeats, a.timeout_ms, a.verbose, a.required_k_tile, a.k_tile_multiplier) == (1, 2, 3, 0, 7, 0, 2, 8, 3, 500, 0, 0, 0)
    assert lib.rk_npu_strerror(0) == b"ok" and lib.rk_npu_strerror(-6) and lib.rk_npu_strerror(-99) == b"unknown error"


def test_memory_query_known_answers(lib):
    # tests/test_w4a8_cpu.cpp:143-152
    info = W4A8MemoryInfo()
    assert lib.rk_npu_w4a8_memory_query(C.byref(cfg_of(lib, 3, 65, 513)), C.byref(info)) == 0
    assert info.weight_metadata_bytes == 520 and info.cpu_scratch_bytes == 3 * 128 * 4 + 3 * 8
    assert lib.rk_npu_w4a8_memory_query(None, C.byref(info)) == -3
    assert lib.rk_npu_w4a8_memory_query(C.byref(cfg_of(lib, 3, 65, 513)), None) == -3
    # tests/test_w4a8_reduction.cpp:112-119
    assert lib.rk_npu_w4a8_memory_query(C.byref(cfg_of(lib, 128, 4096, 11008)), C.byref(info)) == 0
    assert info.backend.partial_bytes == 2 * 128 * 4096 * 4
    # tests/test_w4a8_chain.cpp:46-50: all-K chain keeps every wave's partials
    for M in (1, 2, 4, 8):
        c = cfg_of(lib, M, 193, 1057, pipeline=capi.RK_NPU_W4A8_CHAIN)
        assert lib.rk_npu_w4a8_memory_query(C.byref(c), C.byref(info)) == 0
        assert info.backend.input_bytes == M * 1088 and info.backend.partial_bytes == 3 * 4 * M * 256
    # weight bytes, tests/test_i4_cpu.cpp:43-47 (K513 N65 -> 544 x 128 / 2)
    size = C.c_uint64()
    assert lib.rk_npu_i4_weights_memory_query(C.byref(I4WeightConfig(513, 65, 480)), C.byref(size)) == 0
    assert size.value == 34816
    assert lib.rk_npu_i4_weights_memory_query(C.byref(I4WeightConfig(513, 65, 31)), C.byref(size)) == -3


def test_memory_query_param_matrix(lib):
    ok = cfg_of(lib, 5, 129, 1025)
    ex = W4A8MemoryInfoEx()
    assert lib.rk_npu_w4a8_memory_query_ex(C.byref(ok), None, C.byref(ex)) == 0
    bad = dict(M=0, N=0, K=0, m_tile=0, k_tile=0, n_tile=32, npu_core_mask=5, timeout_ms=0, pipeline=3, cpu_threads=5)
    for field, value in bad.items():
        c = cfg_of(lib, 5, 129, 1025, **{field: value})
        assert lib.rk_npu_w4a8_memory_query_ex(C.byref(c), None, C.byref(ex)) == -3, field
    for field, value in dict(m_tile=65, k_tile=2080, n_tile=8192, K=(2 ** 31 - 1) // 1024 + 1).items():
        c = cfg_of(lib, 5, 129, 1025, **{field: value})
        assert lib.rk_npu_w4a8_memory_query_ex(C.byref(c), None, C.byref(ex)) == -3, field
    assert lib.rk_npu_w4a8_memory_query_ex(C.byref(cfg_of(lib, 5, 64, 1025, npu_core_mask=7)), None, C.byref(ex)) == -3
    o = W4A8Options()
    lib.rk_npu_w4a8_options_init(C.byref(o))
    o.struct_size = 4
    assert lib.rk_npu_w4a8_memory_query_ex(C.byref(ok), C.byref(o), C.byref(ex)) == -3
    lib.rk_npu_w4a8_options_init(C.byref(o))
    o.reduce_backend = 1
    assert lib.rk_npu_w4a8_memory_query_ex(C.byref(cfg_of(lib, 16, 129, 1025)), C.byref(o), C.byref(ex)) == 0
    assert ex.effective_reduce_backend == 0       # M <= 16 falls back to the CPU-reduce policy
    assert lib.rk_npu_w4a8_memory_query_ex(C.byref(cfg_of(lib, 33, 64, 480)), C.byref(o), C.byref(ex)) == 0
    assert ex.effective_reduce_backend == 1 and ex.reduction_control_bytes == 584
    c = cfg_of(lib, 33, 64, 480, pipeline=capi.RK_NPU_W4A8_CHAIN)
    assert lib.rk_npu_w4a8_memory_query_ex(C.byref(c), C.byref(o), C.byref(ex)) == -3   # chain + NPU reduce


def _fields(s):
    out = []
    for name, _ in s._fields_:
        v = getattr(s, name)
        out.extend(_fields(v) if isinstance(v, C.Structure) else [v])
    return out


def test_memory_query_equals_reference_build(lib, reference):
    ref = reference.lib
    rng = np.random.Generator(np.random.PCG64(7))
    checked = accepted = 0
    for _ in range(4000):
        M = int(rng.choice([1, 2, 3, 8, 16, 17, 33, 64, 65, 128, 129, 257, 1024]))
        N = int(rng.choice([1, 64, 65, 129, 193, 256, 1025, 4096, 11008]))
        K = int(rng.choice([1, 33, 480, 513, 1025, 2049, 4096, 20003]))
        c = cfg_of(lib, M, N, K, m_tile=int(rng.choice([1, 3, 4, 8, 16, 64, 65, 128, 256, 257])),
                   k_tile=int(rng.choice([32, 256, 480, 992, 2048, 2080, 100])),
                   n_tile=int(rng.choice([64, 128, 1024, 1408, 8128, 8192, 96])),
                   npu_core_mask=int(rng.choice([1, 2, 3, 4, 7, 5])), pipeline=int(rng.integers(0, 4)),
                   cpu_threads=int(rng.integers(0, 6)))
        o = W4A8Options(C.sizeof(W4A8Options), int(rng.integers(0, 2)), int(rng.integers(0, 2)))
        mine, theirs = W4A8MemoryInfoEx(), W4A8MemoryInfoEx()
        rc_mine = lib.rk_npu_w4a8_memory_query_ex(C.byref(c), C.byref(o), C.byref(mine))
        rc_ref = ref.rk_npu_w4a8_memory_query_ex(C.byref(c), C.byref(o), C.byref(theirs))
        assert rc_mine == rc_ref, (_fields(c), _fields(o), rc_mine, rc_ref)
        if rc_ref == 0:
            assert _fields(mine) == _fields(theirs), (_fields(c), _fields(o))
            accepted += 1
        checked += 1
    assert accepted > 200 and checked == 4000


# ------------------------------------------------------------------ tuning cache
def _affinity_first(n):
    cpus = sorted(os.sched_getaffinity(0))
    order = [c for c in range(4, 8) if c in cpus] + [c for c in cpus if c < 4 or c > 7]
    return sum(1 << c for c in order[:n] if c < 64), min(n, len(order))


def _strategy(lib, ctx, c, B, sw, k_tile, safe, fingerprint, m_tile=64, layout=0):
    cpu_mask, threads = _affinity_first(4)
    s = W4A8StrategyEx()
    s.base.config = cfg_of(lib, c.M, c.N, c.K, m_tile=m_tile, k_tile=k_tile, n_tile=256, npu_core_mask=7,
                           timeout_ms=c.timeout_ms, pipeline=1, cpu_threads=threads)
    s.base.activation_type = c.activation_type
    s.base.cpu_core_mask = cpu_mask
    s.base.weights.config = I4WeightConfig(c.K, c.N, k_tile)
    s.base.weights.safe_k_tile = safe
    s.base.weights.multiplier = 1.0
    s.base.weights.bound_relaxed = 0
    s.base.weight_fingerprint = fingerprint
    s.base.tuning_revision = 5
    s.base.total_us, s.base.robust_us = 1.25, 1.5
    s.execution = W4A8Options(C.sizeof(W4A8Options), layout, 0)
    return s


@pytest.fixture()
def cache_case(lib, oracle, tmp_path, monkeypatch):
    monkeypatch.delenv("RK_NPU_W4A8_CHAIN_MAX_M", raising=False)
    monkeypatch.delenv("RK_NPU_W4A8_K_TILE_MULTIPLIER", raising=False)
    ctx = lib.rk_npu_b200_open_offline(0x908)
    assert ctx and lib.rk_npu_b200_device(ctx) == -1
    assert not lib.rk_npu_iommu_domain_create(ctx, 0)     # an offline context can do no device work
    c = W4A8AutotuneConfig()
    lib.rk_npu_w4a8_autotune_config_init(C.byref(c), 128, 193, 2048)
    c.k_tile_multiplier = 1.0
    c.required_k_tile = 2048
    B = np.ones((c.K, c.N), np.int8)
    sw = np.full(c.N, .125, np.float32)
    rc, safe, _, _, mask = oracle.bound(B)
    assert rc == 0 and safe == 2048
    s = _strategy(lib, ctx, c, B, sw, 2048, safe, oracle.fingerprint(B, sw), m_tile=128, layout=1)
    yield lib, ctx, c, B, sw, s, str(tmp_path / "entry.tune")
    lib.rk_npu_close(ctx)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def test_cache_round_trip_and_invalidation(cache_case):
    lib, ctx, c, B, sw, s, path = cache_case
    p = path.encode()
    f, st = W4A8StrategyEx(), W4A8StrategyEx()
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == -9   # absent
    assert lib.rk_npu_w4a8_autotune_cache_save_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(s), C.byref(s)) == 0
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == 0
    assert f.execution.input_layout == 1 and f.base.config.m_tile == 128 and f.base.total_us == 1.25
    assert _fields(f) == _fields(s) and _fields(st) == _fields(s)
    lines = Path(path).read_text().splitlines()
    assert lines[0] == "rk_npu_w4a8_tuning_cache_v2" and lines[2].startswith("fastest ") and lines[3].startswith("stable ")
    assert lines[1].split()[:7] == ["5", "3", str(0x908), "128", "193", "2048", "0"]
    # the native-only (legacy) lookup uses another search-space id and must miss
    lf, ls = W4A8Strategy(), W4A8Strategy()
    assert lib.rk_npu_w4a8_autotune_cache_load(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(lf), C.byref(ls)) == -9
    # every key component invalidates: weights, scales, shape, measurement settings, dtype
    B2 = B.copy(); B2[5, 5] = 2
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B2), _p(sw), p, C.byref(f), C.byref(st)) == -9
    sw2 = sw.copy(); sw2[0] = .25
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw2), p, C.byref(f), C.byref(st)) == -9
    for field, value in dict(loops=9, warmup=3, repeats=4, timeout_ms=400, activation_type=1).items():
        c2 = W4A8AutotuneConfig.from_buffer_copy(c)
        setattr(c2, field, value)
        assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c2), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == -9, field
    other = lib.rk_npu_b200_open_offline(0x909)      # another driver version
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(other, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == -9
    lib.rk_npu_close(other)
    # trailing bytes, an old magic line
    text = Path(path).read_text()
    Path(path).write_text(text + "junk\n")
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == -9
    Path(path).write_text(text.replace("cache_v2", "cache_v1", 1))
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == -9
    Path(path).write_text(text)
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == 0


def test_cache_rejects_invalid_strategies(cache_case):
    lib, ctx, c, B, sw, s, path = cache_case
    p = path.encode()
    for mutate in ("layout", "reduce", "size", "revision", "threads", "pipeline", "fingerprint", "ktile"):
        bad = W4A8StrategyEx.from_buffer_copy(s)
        if mutate == "layout": bad.execution.input_layout = 7
        if mutate == "reduce": bad.execution.reduce_backend = 1
        if mutate == "size": bad.execution.struct_size = 0
        if mutate == "revision": bad.base.tuning_revision = 4
        if mutate == "threads": bad.base.config.cpu_threads = 3 if s.base.config.cpu_threads != 3 else 2
        if mutate == "pipeline": bad.base.config.pipeline = 3
        if mutate == "fingerprint": bad.base.weight_fingerprint ^= 1
        if mutate == "ktile": bad.base.config.k_tile = 480
        assert lib.rk_npu_w4a8_autotune_cache_save_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(bad), C.byref(bad)) == -3, mutate
    assert lib.rk_npu_w4a8_autotune_cache_save_ex(ctx, C.byref(c), _p(B), _p(sw), b"", C.byref(s), C.byref(s)) == -3
    assert lib.rk_npu_w4a8_autotune_cache_save_ex(None, C.byref(c), _p(B), _p(sw), p, C.byref(s), C.byref(s)) == -3


def test_cache_environment_is_part_of_the_key(cache_case, monkeypatch):
    lib, ctx, c, B, sw, s, path = cache_case
    p = path.encode()
    f, st = W4A8StrategyEx(), W4A8StrategyEx()
    assert lib.rk_npu_w4a8_autotune_cache_save_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(s), C.byref(s)) == 0
    for value in ("0", "2", "16", "64"):
        monkeypatch.setenv("RK_NPU_W4A8_CHAIN_MAX_M", value)
        assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == -9
    for value in ("", "-1", "65", "eight", "99999999999999999"):
        monkeypatch.setenv("RK_NPU_W4A8_CHAIN_MAX_M", value)
        assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == -3
    monkeypatch.setenv("RK_NPU_W4A8_CHAIN_MAX_M", "8")
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), p, C.byref(f), C.byref(st)) == 0


def test_cache_files_interoperate_with_reference_build(cache_case, reference, tmp_path):
    """A file written by this library is a hit for the reference's loader and the reverse."""
    lib, ctx, c, B, sw, s, path = cache_case
    ref = reference.lib
    # the reference's context object: fd at offset 0, driver version at offset 16
    fake = (C.c_uint8 * 8192)()
    C.cast(fake, C.POINTER(C.c_int))[0] = -1
    C.cast(C.byref(fake, 16), C.POINTER(C.c_uint32))[0] = 0x908
    f, st = W4A8StrategyEx(), W4A8StrategyEx()
    assert lib.rk_npu_w4a8_autotune_cache_save_ex(ctx, C.byref(c), _p(B), _p(sw), path.encode(), C.byref(s), C.byref(s)) == 0
    assert ref.rk_npu_w4a8_autotune_cache_load_ex(fake, C.byref(c), _p(B), _p(sw), path.encode(), C.byref(f), C.byref(st)) == 0
    assert _fields(f) == _fields(s)
    theirs = str(tmp_path / "theirs.tune").encode()
    assert ref.rk_npu_w4a8_autotune_cache_save_ex(fake, C.byref(c), _p(B), _p(sw), theirs, C.byref(s), C.byref(s)) == 0
    f2, st2 = W4A8StrategyEx(), W4A8StrategyEx()
    assert lib.rk_npu_w4a8_autotune_cache_load_ex(ctx, C.byref(c), _p(B), _p(sw), theirs, C.byref(f2), C.byref(st2)) == 0
    assert _fields(f2) == _fields(s)
    assert Path(path).read_bytes() == Path(theirs.decode()).read_bytes()


# ---------------------------------------------------------------- the rest of the original headers
def test_every_entry_point_of_the_original_headers_links(lib):
    # tests/golden/reference_header_symbols.txt (written by tests/golden/abi_layout.py --symbols): every function the
    # seven public headers of the path declare (rk_npu_common.h, rk_npu_matmul_i4.h, rk_npu_w4a8.h, rk_npu_w4a8_tune.h,
    # rk_npu_quant_matmul.h, rk_npu_moe_w8.h, rk_npu_add_rmsnorm_f16.h)
    names = (ROOT / "tests" / "golden" / "reference_header_symbols.txt").read_text().split()
    assert len(names) == 125
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # operators that are not built decline instead of pretending
    for name in ("rk_npu_i8i8i32_autotune", "rk_npu_f16i8f16_dynamic_autotune_family",
                 "rk_npu_matmul_autotune_family_cached", "rk_npu_matmul_autotune_cached"):
        fn = C.CDLL(str(capi.LIB_PATH))[name]
        fn.restype, fn.argtypes = C.c_int, []
        assert fn() == capi.RK_NPU_ERR_PARAM, name
    for name in ("rk_npu_f32i8f32_weights_create_from_f32_compress", "rk_npu_f16i8f16_weights_create_from_f32_compress"):
        fn = C.CDLL(str(capi.LIB_PATH))[name]
        fn.restype, fn.argtypes = C.c_void_p, []
        assert fn() is None, name
    # the compressed-storage constructors are the plain ones here: argument errors are answered alike
    assert lib.rk_npu_i8i8i32_weights_create_compress(None, None, None) is None
    assert lib.rk_npu_f16i8f16_weights_create_compress(None, None, None, None) is None
    assert lib.rk_npu_f32i8f32_weights_compressed_layout_generation(None) == 0
    # the typed W8A8 operators are built: argument errors are answered as such, without a device
    assert lib.rk_npu_i8i8i32_run(None, None, None, None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_f16i8f16_run_static(None, None, None, None, None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_matmul_workspace_create(None, None) is None
    assert lib.rk_npu_f32i8f32_weights_create(None, None, None, None) is None
    # so is the exact int4 operator
    assert lib.rk_npu_i4i4i32_run(None, None, None, None, None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_i4_workspace_create(None, None) is None and lib.rk_npu_i4i4i32_weights_create(None, None, None) is None
    # the search tuners are built: argument errors are answered as such, without a device
    fast = capi.W4A8Strategy()
    assert lib.rk_npu_w4a8_autotune(None, None, None, None, C.byref(fast), None) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_w4a8_autotune_cached(None, None, None, None, None, 0, C.byref(fast), None, None) == capi.RK_NPU_ERR_PARAM


def test_second_header_defaults(lib):
    c = capi.MatmulAutotuneConfig()
    lib.rk_npu_matmul_autotune_config_init(C.byref(c), 5, 6, 7)
    assert (c.M, c.N, c.K, c.allowed_npu_core_mask, c.allowed_cpu_core_mask, c.warmup, c.loops, c.repeats, c.timeout_ms,
            c.verbose, c.required_k_tile) == (5, 6, 7, 7, 0, 2, 8, 3, 500, 0, 0)
    ms = (C.c_int * 3)(1, 8, 32)
    f = capi.MatmulFamilyAutotuneConfig()
    lib.rk_npu_matmul_family_autotune_config_init(C.byref(f), 64, 96, 3, ms)
    assert (f.K, f.N, f.m_count, f.allowed_npu_core_mask, f.warmup, f.loops, f.repeats, f.timeout_ms) == (96, 64, 3, 7, 2, 8, 3, 500)
    i4 = capi.I4Config()
    lib.rk_npu_i4_config_init(C.byref(i4), 3, 4, 5)
    assert (i4.M, i4.N, i4.K, i4.m_tile, i4.k_tile, i4.n_tile, i4.npu_core_mask, i4.timeout_ms, i4.pipeline,
            i4.cpu_threads) == (3, 4, 5, 128, 480, 1024, 1, 500, 1, 1)
    fam = capi.W4A8FamilyConfig()
    lib.rk_npu_w4a8_family_config_init(C.byref(fam), 64, 96, 3, ms)
    assert (fam.base.M, fam.base.N, fam.base.K, fam.m_count, fam.base.loops) == (1, 64, 96, 3, 8)


def _w8_file(path, key, fastest, stable, magic="rk_npu_matmul_tuning_cache_v2"):
    # text layout of src/rk_npu_quant_matmul.cpp:252-262,336-347: doubles travel as their 64-bit patterns
    def bits(x):
        return str(np.float64(x).view(np.uint64))

    def record(label, s):
        return " ".join([label] + [str(v) for v in s[:13]] + [bits(v) for v in s[13:]])

    Path(path).write_text(magic + "\n" + "key " + " ".join(str(v) for v in key) + "\n" + record("fastest", fastest) + "\n"
                          + record("stable", stable) + "\n")


def _w8_record(s):
    """A MatmulStrategy as the list of values _w8_file writes."""
    return [s.op_kind, s.M, s.N, s.K, s.k_tile, s.n_tile, s.a_layout, s.c_layout, s.wave_count, s.n_groups, s.npu_core_mask,
            s.cpu_core_mask, s.cpu_threads, s.input_us, s.npu_us, s.sync_us, s.output_us, s.total_us, s.jitter_pct, s.robust_us]


def test_w8_cache_load_and_save(lib, tmp_path, monkeypatch):
    import os
    monkeypatch.delenv("RK_NPU_I8_NPU_REDUCE", raising=False)
    monkeypatch.delenv("RK_NPU_W8A8_NPU_DEQUANT", raising=False)
    ctx = lib.rk_npu_b200_open_offline(0x908)
    c = capi.MatmulAutotuneConfig()
    lib.rk_npu_matmul_autotune_config_init(C.byref(c), 128, 4096, 11008)
    affinity = 0
    for cpu in os.sched_getaffinity(0):
        if cpu < 64:
            affinity |= 1 << cpu
    cpu_mask = affinity & -affinity                      # one permitted CPU
    kind = 1                                             # RK_NPU_MATMUL_F16I8F16_DYNAMIC
    key = [2, 6, 0x908, kind, 128, 4096, 11008, 7, affinity, 2, 8, 3, 500, 0]
    #        op    M    N     K      kt    nt  a  c  waves        groups  npu cpu       thr  seven timings
    rec = [kind, 128, 4096, 11008, 1376, 1408, 1, 0, 8, -(-4096 // 1408), 7, cpu_mask, 1, 10.5, 200.25, 3.0, 40.0, 250.75, 1.5, 260.0]
    path = str(tmp_path / "w8.tune")
    f, s = capi.MatmulStrategy(), capi.MatmulStrategy()

    def load(cfg=c, k=kind, context=ctx):
        return lib.rk_npu_matmul_autotune_cache_load(context, path.encode(), k, C.byref(cfg), C.byref(f), C.byref(s))

    assert load() == capi.RK_NPU_ERR_CACHE_MISS          # absent
    _w8_file(path, key, rec, rec)
    assert load() == 0
    assert (f.op_kind, f.M, f.N, f.K, f.k_tile, f.n_tile, f.a_layout, f.c_layout, f.wave_count, f.n_groups, f.npu_core_mask,
            f.cpu_core_mask, f.cpu_threads) == tuple(rec[:6] + [1, 0] + rec[8:13])
    assert (f.input_us, f.npu_us, f.sync_us, f.output_us, f.total_us, f.jitter_pct, f.robust_us) == tuple(rec[13:])
    assert s.total_us == 250.75
    # arguments
    assert lib.rk_npu_matmul_autotune_cache_load(ctx, b"", kind, C.byref(c), C.byref(f), C.byref(s)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_matmul_autotune_cache_load(ctx, path.encode(), 9, C.byref(c), C.byref(f), C.byref(s)) == capi.RK_NPU_ERR_PARAM
    bad = capi.MatmulAutotuneConfig.from_buffer_copy(c); bad.loops = 0
    assert load(bad) == capi.RK_NPU_ERR_PARAM
    # every key component invalidates
    for field, value in dict(M=64, loops=9, warmup=3, repeats=4, timeout_ms=400, required_k_tile=32, allowed_npu_core_mask=3).items():
        c2 = capi.MatmulAutotuneConfig.from_buffer_copy(c)
        setattr(c2, field, value)
        assert load(c2) == capi.RK_NPU_ERR_CACHE_MISS, field
    assert load(k=2) == capi.RK_NPU_ERR_CACHE_MISS       # another operator
    other = lib.rk_npu_b200_open_offline(0x909)
    assert load(context=other) == capi.RK_NPU_ERR_CACHE_MISS
    lib.rk_npu_close(other)
    monkeypatch.setenv("RK_NPU_I8_NPU_REDUCE", "1")      # the execution mode is part of the stored revision
    assert load() == capi.RK_NPU_ERR_CACHE_MISS
    monkeypatch.delenv("RK_NPU_I8_NPU_REDUCE")
    assert load() == 0
    # stale files and invalid records
    for k2 in ([2, 5] + key[2:], [1] + key[1:]):
        _w8_file(path, k2, rec, rec)
        assert load() == capi.RK_NPU_ERR_CACHE_MISS
    _w8_file(path, key, rec, rec, magic="rk_npu_matmul_tuning_cache_v1")
    assert load() == capi.RK_NPU_ERR_CACHE_MISS
    for index, value in ((4, 20000), (5, 1400), (5, 3104), (8, 7), (9, 2), (10, 5), (12, 2), (7, 2), (7, 1), (17, -1.0),
                         (15, float("nan"))):     # (7, 1), (7, 2): panels of C need a normal or a panel A, this record's is native
        r2 = list(rec)
        r2[index] = value
        _w8_file(path, key, rec, r2)
        assert load() == capi.RK_NPU_ERR_CACHE_MISS, (index, value)
    # panel recipes are hits where the original's device plan takes them: 8-row panels of A (128 rows, K tile 1376)
    r2 = list(rec)
    r2[6] = 2
    _w8_file(path, key, rec, r2)
    assert load() == 0 and s.a_layout == 2
    r2[6], r2[7] = 0, 1                                  # a normal A with 8-row panels of C
    _w8_file(path, key, rec, r2)
    assert load() == 0 and (s.a_layout, s.c_layout) == (0, 1)
    # save: what was loaded goes back out as the same text; arguments and records are checked first
    _w8_file(path, key, rec, rec)
    assert load() == 0
    out_path = str(tmp_path / "saved.tune").encode()
    assert lib.rk_npu_matmul_autotune_cache_save(ctx, out_path, kind, C.byref(c), C.byref(f), C.byref(s)) == 0
    assert Path(out_path.decode()).read_text() == Path(path).read_text()
    assert lib.rk_npu_matmul_autotune_cache_save(ctx, b"", kind, C.byref(c), C.byref(f), C.byref(s)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_matmul_autotune_cache_save(ctx, None, kind, C.byref(c), C.byref(f), C.byref(s)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_matmul_autotune_cache_save(None, out_path, kind, C.byref(c), C.byref(f), C.byref(s)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_matmul_autotune_cache_save(ctx, out_path, kind, C.byref(c), None, C.byref(s)) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_matmul_autotune_cache_save(ctx, out_path, 2, C.byref(c), C.byref(f), C.byref(s)) == capi.RK_NPU_ERR_PARAM      # another operator
    wrong = capi.MatmulStrategy.from_buffer_copy(f)
    wrong.wave_count += 1
    assert lib.rk_npu_matmul_autotune_cache_save(ctx, out_path, kind, C.byref(c), C.byref(wrong), C.byref(s)) == capi.RK_NPU_ERR_PARAM
    wrong = capi.MatmulStrategy.from_buffer_copy(f)
    wrong.total_us = float("nan")
    assert lib.rk_npu_matmul_autotune_cache_save(ctx, out_path, kind, C.byref(c), C.byref(f), C.byref(wrong)) == capi.RK_NPU_ERR_PARAM
    blocked = tmp_path / "file_not_dir"
    blocked.write_text("x")
    assert lib.rk_npu_matmul_autotune_cache_save(ctx, str(blocked / "a.tune").encode(), kind, C.byref(c), C.byref(f), C.byref(s)) == capi.RK_NPU_ERR_IO
    _w8_file(path, key, rec, rec)
    Path(path).write_text(Path(path).read_text() + "junk\n")
    assert load() == capi.RK_NPU_ERR_CACHE_MISS          # trailing bytes
    lib.rk_npu_close(ctx)


def test_w8_cache_files_written_by_the_reference_load_here(lib, reference, tmp_path, monkeypatch):
    """Files written by the reference's own W8 cache writer (src/rk_npu_quant_matmul.cpp:337-349, compiled into the
    reference checker) are hits for this library's loader with identical records, and misses for every other key.
    Records that name a panel layout are accepted by the reference after a check against its device plan
    (src/rk_npu_quant_matmul.cpp:167-177); this library restates that check, and the two sides agree on every
    combination of layouts over a grid of shapes: what the reference's writer refuses or its loader misses, this
    loader misses, and what it accepts is a hit with the same record."""
    import os
    ref = reference.lib
    if not hasattr(ref, "rk_npu_matmul_autotune_cache_save"):
        pytest.skip("reference checker built without its W8 sources")
    monkeypatch.delenv("RK_NPU_I8_NPU_REDUCE", raising=False)
    monkeypatch.delenv("RK_NPU_W8A8_NPU_DEQUANT", raising=False)
    fake = (C.c_uint8 * 8192)()                                     # the reference's context: fd at 0, driver version at 16
    C.cast(fake, C.POINTER(C.c_int))[0] = -1
    C.cast(C.byref(fake, 16), C.POINTER(C.c_uint32))[0] = 0x908
    ctx = lib.rk_npu_b200_open_offline(0x908)
    affinity = sum(1 << cpu for cpu in os.sched_getaffinity(0) if cpu < 64)
    one_cpu = affinity & -affinity
    for kind, (M, N, K), kt, nt in ((1, (128, 4096, 11008), 1376, 1408), (0, (8, 1000, 513), 513, 512), (3, (33, 4096, 4096), 2048, 2048)):
        c = capi.MatmulAutotuneConfig()
        lib.rk_npu_matmul_autotune_config_init(C.byref(c), M, N, K)
        s = capi.MatmulStrategy()
        s.op_kind, s.M, s.N, s.K, s.k_tile, s.n_tile = kind, M, N, K, kt, nt
        s.a_layout, s.c_layout = 1, 0
        s.wave_count = -(-K // kt)
        s.n_groups = -(-max(32, -(-N // 32) * 32) // nt)
        s.npu_core_mask, s.cpu_core_mask, s.cpu_threads = 7 if s.n_groups >= 3 else 1, one_cpu, 1
        s.input_us, s.npu_us, s.sync_us, s.output_us, s.total_us, s.jitter_pct, s.robust_us = 1.5, 20.25, 3.0, 4.0, 30.0, 2.0, 31.0
        path = str(tmp_path / f"ref_w8_{kind}.tune").encode()
        assert ref.rk_npu_matmul_autotune_cache_save(fake, path, kind, C.byref(c), C.byref(s), C.byref(s)) == 0
        mine = str(tmp_path / "deep" / "er" / f"mine_w8_{kind}.tune").encode()       # missing directories are made
        assert lib.rk_npu_matmul_autotune_cache_save(ctx, mine, kind, C.byref(c), C.byref(s), C.byref(s)) == 0
        assert Path(mine.decode()).read_bytes() == Path(path.decode()).read_bytes()    # the same bytes as the reference's writer
        assert not [x.name for x in Path(mine.decode()).parent.iterdir() if not x.name.endswith(".tune")]     # no scratch file left
        f, st = capi.MatmulStrategy(), capi.MatmulStrategy()
        assert ref.rk_npu_matmul_autotune_cache_load(fake, mine, kind, C.byref(c), C.byref(f), C.byref(st)) == 0 and _fields(f) == _fields(s)
        assert lib.rk_npu_matmul_autotune_cache_load(ctx, path, kind, C.byref(c), C.byref(f), C.byref(st)) == 0
        assert _fields(f) == _fields(s) and _fields(st) == _fields(s)
        f2, st2 = capi.MatmulStrategy(), capi.MatmulStrategy()
        assert ref.rk_npu_matmul_autotune_cache_load(fake, path, kind, C.byref(c), C.byref(f2), C.byref(st2)) == 0
        c2 = capi.MatmulAutotuneConfig.from_buffer_copy(c)
        c2.loops += 1
        assert lib.rk_npu_matmul_autotune_cache_load(ctx, path, kind, C.byref(c2), C.byref(f), C.byref(st)) == capi.RK_NPU_ERR_CACHE_MISS
        assert ref.rk_npu_matmul_autotune_cache_load(fake, path, kind, C.byref(c2), C.byref(f2), C.byref(st2)) == capi.RK_NPU_ERR_CACHE_MISS

    # panel recipes: every (a_layout, c_layout) pair over shapes on both sides of each bound
    accepted = refused = 0
    kind = 1
    shapes = [(128, 4096, 4096, 1024), (128, 4096, 4096, 2048), (128, 4096, 4096, 2080), (128, 4096, 8192, 4096), (128, 4096, 8320, 4128),
              (128, 4096, 16384, 8192), (128, 4096, 16640, 8224), (12, 256, 512, 512), (24, 256, 512, 256), (48, 4096, 1024, 1024),
              (64, 32768, 256, 256), (64, 65568, 256, 256), (64, 16416, 256, 256), (7, 64, 64, 64), (16, 131072, 64, 64)]
    for M, N, K, kt in shapes:
        for a_layout in range(4):
            for c_layout in range(3):
                c = capi.MatmulAutotuneConfig()
                lib.rk_npu_matmul_autotune_config_init(C.byref(c), M, N, K)
                s = capi.MatmulStrategy()
                nt = min(2048, max(32, -(-N // 32) * 32))
                s.op_kind, s.M, s.N, s.K, s.k_tile, s.n_tile = kind, M, N, K, kt, nt
                s.a_layout, s.c_layout = a_layout, c_layout
                s.wave_count = -(-K // kt)
                s.n_groups = -(-max(32, -(-N // 32) * 32) // nt)
                s.npu_core_mask, s.cpu_core_mask, s.cpu_threads = 1, one_cpu, 1
                s.input_us, s.npu_us, s.sync_us, s.output_us, s.total_us, s.jitter_pct, s.robust_us = 1.5, 20.25, 3.0, 4.0, 30.0, 2.0, 31.0
                plain = capi.MatmulStrategy.from_buffer_copy(s)
                plain.a_layout, plain.c_layout = 1, 0
                path = str(tmp_path / f"panel_{M}_{N}_{K}_{kt}_{a_layout}_{c_layout}.tune").encode()
                saved = ref.rk_npu_matmul_autotune_cache_save(fake, path, kind, C.byref(c), C.byref(plain), C.byref(s))
                mine = path + b".mine"
                assert lib.rk_npu_matmul_autotune_cache_save(ctx, mine, kind, C.byref(c), C.byref(plain), C.byref(s)) == saved
                if saved == 0:
                    assert Path(mine.decode()).read_bytes() == Path(path.decode()).read_bytes()
                else:
                    assert not Path(mine.decode()).exists()
                f, st, f2, st2 = (capi.MatmulStrategy() for _ in range(4))
                theirs = ref.rk_npu_matmul_autotune_cache_load(fake, path, kind, C.byref(c), C.byref(f2), C.byref(st2)) if saved == 0 else saved
                if saved != 0:      # the writer refuses the recipe: the same file written by hand must be a miss here too
                    key = [2, 6, 0x908, kind, M, N, K, c.allowed_npu_core_mask, affinity, c.warmup, c.loops, c.repeats, c.timeout_ms, 0]
                    _w8_file(path.decode(), key, _w8_record(plain), _w8_record(s))
                ours = lib.rk_npu_matmul_autotune_cache_load(ctx, path, kind, C.byref(c), C.byref(f), C.byref(st))
                assert (ours == 0) == (theirs == 0), (M, N, K, kt, a_layout, c_layout, ours, theirs)
                if ours == 0:
                    accepted += 1
                    assert _fields(st) == _fields(s) == _fields(st2)
                else:
                    refused += 1
    assert accepted >= 40 and refused >= 60, (accepted, refused)
    lib.rk_npu_close(ctx)


def test_public_headers_are_valid_c(tmp_path):
    # the original checks its headers with a C translation unit (tests/test_w4a8_header.c, tests/test_quant_header.c)
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if not gcc:
        pytest.skip("no C compiler")
    src = tmp_path / "headers.c"
    src.write_text('#include "rknpu_b200_w4a8.h"\n#include "rknpu_b200_quant.h"\n#include "rknpu_b200_moe.h"\n#include "rknpu_b200_rmsnorm.h"\n#include "rknpu_b200_ext.h"\n'
                   "int main(void) { rk_npu_w4a8_config c; rk_npu_matmul_strategy s; rk_npu_moe_w8_config m; (void)c; (void)s; (void)m; return 0; }\n")
    out = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", f"-I{ROOT / 'include'}",
                          str(src)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr


def test_the_original_example_programs_link_unchanged(lib, tmp_path):
    # examples/tune_w4a8.cpp (the search tuner's command-line front end), examples/bench_w4a8.cpp and examples/bench_i4.cpp of
    # the original use only the public headers of this path (bench_w4a8 also its header-only binary16 helpers): compiled
    # from where they lie and linked against this library instead of librk_npu_matmul.so, every symbol resolves
    import shutil
    import subprocess
    default = re.search(r"^REF\s*\?=\s*(\S+)", (ROOT / "oracle" / "Makefile").read_text(), flags=re.M).group(1)
    tree = Path(os.environ.get("REF", default))
    gxx = shutil.which("g++")
    if not gxx or not (tree / "examples" / "tune_w4a8.cpp").exists():
        pytest.skip("needs g++ and the original tree")
    for name in ("tune_w4a8", "bench_w4a8", "bench_i4"):
        out = subprocess.run([gxx, "-O1", "-std=c++17", f"-I{tree / 'include'}", "-o", str(tmp_path / name), str(tree / "examples" / f"{name}.cpp"),
                              f"-L{capi.LIB_PATH.parent}", "-lrk_npu_matmul_b200", "-Wl,--no-undefined"], capture_output=True, text=True)
        assert out.returncode == 0, f"{name}: {out.stderr[-2000:]}"


# ---------------------------------------------------------------- exact int4 operator: pure host functions
def test_i4_memory_query_and_tile_packing_match_the_reference(lib):
    from oracle.harness import REF_SO, Reference
    if not Reference.available():
        pytest.skip("reference checker not built")
    ref = C.CDLL(str(REF_SO))
    rng = np.random.default_rng(4)
    cases = [(1, 64, 32, 1, 32, 64, 1, 1, 1), (128, 4096, 4096, 128, 480, 1024, 7, 1, 4), (33, 1000, 513, 16, 2048, 8128, 3, 0, 2),
             (5, 64, 40, 129, 480, 1024, 1, 1, 1), (5, 64, 40, 8, 481, 1024, 1, 1, 1), (5, 64, 40, 8, 480, 100, 1, 1, 1),
             (5, 64, 40, 8, 480, 64, 3, 1, 1), (5, 64, 40, 8, 480, 64, 1, 2, 1), (5, 64, 40, 8, 480, 64, 1, 1, 5), (0, 64, 40, 8, 480, 64, 1, 1, 1)]
    for _ in range(200):
        cases.append((int(rng.integers(1, 600)), int(rng.integers(1, 9000)), int(rng.integers(1, 9000)), int(rng.integers(1, 140)),
                      int(rng.integers(1, 70)) * 32, int(rng.integers(1, 130)) * 64, int(rng.choice([1, 2, 4, 3, 7, 5])),
                      int(rng.integers(0, 2)), int(rng.integers(1, 5))))
    for (M, N, K, mt, kt, nt, mask, pipe, thr) in cases:
        cfg = capi.I4Config(M, N, K, mt, kt, nt, mask, 500, pipe, thr)
        a, b = capi.I4MemoryInfo(), capi.I4MemoryInfo()
        ra = lib.rk_npu_i4_memory_query(C.byref(cfg), C.byref(a))
        rb = ref.rk_npu_i4_memory_query(C.byref(cfg), C.byref(b))
        assert ra == rb, (M, N, K, mt, kt, nt, mask, pipe, thr)
        if ra == 0:
            assert bytes(a) == bytes(b)
    # the reference producer helper: same bytes, same verdicts
    M, K = 37, 300
    A = rng.integers(-8, 8, size=(M, K), dtype=np.int8)
    for (m0, rows, k0, k) in [(0, 37, 0, 300), (5, 16, 32, 200), (36, 1, 288, 12), (0, 128, 0, 10)]:
        padded = (k + 31) // 32 * 32
        outs = []
        for L in (lib, ref):
            buf = np.full(max(rows, 1) * padded // 2 + 8, 0x5A, np.uint8)
            tile = capi.I4InputTile(m0, rows, k0, k, padded, buf.ctypes.data_as(C.POINTER(C.c_uint8)), rows * padded // 2)
            fn = L.rk_npu_i4_pack_a_tile
            fn.restype, fn.argtypes = C.c_int, [C.POINTER(capi.I4InputTile), C.c_void_p, C.c_int]
            rc = fn(C.byref(tile), A.ctypes.data, K) if m0 + rows <= M else capi.RK_NPU_ERR_PARAM
            outs.append((rc, buf.copy()))
        assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1]), (m0, rows, k0, k)
    bad = A.copy()
    bad[3, 17] = 8
    buf = np.zeros(M * 320 // 2, np.uint8)
    tile = capi.I4InputTile(0, M, 0, K, 320, buf.ctypes.data_as(C.POINTER(C.c_uint8)), M * 320 // 2)
    assert lib.rk_npu_i4_pack_a_tile(C.byref(tile), bad.ctypes.data, K) == capi.RK_NPU_ERR_PARAM
    assert lib.rk_npu_i4_pack_a_tile(C.byref(tile), A.ctypes.data, K - 1) == capi.RK_NPU_ERR_PARAM       # lda too small
