import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.harness import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU stages; skipped where they were not built."""
    from oracle.harness import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/librk_npu_ref.so not built (needs the reference tree)")
    return Reference()


@pytest.fixture(scope="session")
def golden_linear():
    return np.load(GOLDEN / "linear_reference.npz")


@pytest.fixture(scope="session")
def golden_ffn():
    return np.load(GOLDEN / "ffn_reference.npz")


@pytest.fixture(scope="session")
def golden_half():
    return np.load(GOLDEN / "half_reference.npz")


@pytest.fixture(scope="session")
def lib():
    from rknpu2_matmul_open_b200 import build, capi
    build.build_library()
    return capi.load()


@pytest.fixture(scope="session")
def gpu():
    """(context, domain 0, domain 1) on cuda:0."""
    import rknpu2_matmul_open_b200 as rk
    ctx = rk.Context("cuda:0")
    d0, d1 = ctx.domain(0), ctx.domain(1)
    yield ctx, d0, d1
    d1.free()
    d0.free()
    ctx.close()


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32}[a.dtype.itemsize])
