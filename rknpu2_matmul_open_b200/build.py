"""Compile the CUDA library in-tree for sm_100a (nvcc cross-compiles without a GPU)."""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB_DIR = HERE / "lib"
LIB = LIB_DIR / "librk_npu_matmul_b200.so"
TOOLS = ["int8_peak.cu"]   # measures the dense int8 tensor peak; bench.py runs it for its roofline denominator
SOURCES = ["w4a8_kernels.cu", "w4a8_fused.cu", "w4a8_decode.cu", "w4a8_stream.cu", "w4a8_shard.cu", "w4a8_gemm_tc.cu", "w4a8_gemm_tc_persist.cu", "w8a8_kernels.cu", "moe_kernels.cu", "rmsnorm_kernels.cu", "w4a8_abi.cpp", "w8a8_abi.cpp", "i4_abi.cpp", "moe_abi.cpp", "rmsnorm_abi.cpp", "w4a8_group.cpp", "w4a8_tune.cpp", "w4a8_autotune.cpp", "w4a8_unbuilt.cpp"]
HEADERS = ["w4a8_device.h", "w4a8_host.h", "w4a8_tune.h", "w4a8_ptx.cuh", "w4a8_math.cuh", "w4a8_tc.cuh", "moe_device.h", "rmsnorm_device.h", "../../include/rknpu_b200_moe.h", "../../include/rknpu_b200_rmsnorm.h", "../../include/rknpu_b200_w4a8.h", "../../include/rknpu_b200_ext.h", "../../include/rknpu_b200_quant.h"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build() -> bool:
    if not LIB.exists():
        return True
    stamp = LIB.stat().st_mtime
    return any((CSRC / f).stat().st_mtime > stamp for f in SOURCES + HEADERS + TOOLS)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Build lib/librk_npu_matmul_b200.so; returns its path. Raises on compiler errors."""
    if not force and not needs_build():
        return LIB
    LIB_DIR.mkdir(exist_ok=True)
    objects = []
    log = []
    def compile_one(src):
        obj = LIB_DIR / (src.rsplit(".", 1)[0] + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", str(CSRC / src), "-o", str(obj)]
        return src, obj, subprocess.run(cmd, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:   # the translation units are independent
        results = list(pool.map(compile_one, SOURCES))
    for src, obj, out in results:
        log.append(out.stderr)
        if out.returncode:
            raise RuntimeError(f"nvcc failed on {src}:\n{out.stdout}\n{out.stderr}")
        objects.append(str(obj))
    link = [_nvcc(), "-shared", "-o", str(LIB), *objects, "-cudart", "static", "-ldl", "-Xlinker", "-Bsymbolic",
            "-Xlinker", f"--version-script={CSRC / 'exports.map'}", "-lpthread"]
    out = subprocess.run(link, capture_output=True, text=True)
    if out.returncode:
        raise RuntimeError(f"link failed:\n{out.stdout}\n{out.stderr}")
    for tool in TOOLS:   # stand-alone measurement program (roofline denominator)
        out = subprocess.run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-o",
                              str(LIB_DIR / tool.rsplit(".", 1)[0]), str(CSRC / tool)], capture_output=True, text=True)
        if out.returncode:
            raise RuntimeError(f"nvcc failed on {tool}:\n{out.stderr}")
    (LIB_DIR / "ptxas.log").write_text("\n".join(log))
    if verbose:
        print("\n".join(log))
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
