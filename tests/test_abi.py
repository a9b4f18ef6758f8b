"""The C-ABI library loads without a GPU and exports every symbol include/muser_cuda.h declares."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from muser_b200 import build
    build.build()
    from muser_b200 import _lib
    return _lib


def test_every_declared_symbol_is_exported(lib):
    header = (ROOT / "include" / "muser_cuda.h").read_text()
    declared = sorted(set(re.findall(r"MUSER_CUDA_API[^;]*?\b(muser_cuda_\w+)\s*\(", header)))
    assert len(declared) >= 18
    assert sorted(lib.EXPORTS) == declared
    raw = C.CDLL(str(lib.LIB_PATH))
    for name in declared:
        assert hasattr(raw, name), name


def test_only_the_abi_is_exported(lib):
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", str(lib.LIB_PATH)], capture_output=True, text=True).stdout
    names = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert names and all(n.startswith("muser_cuda_") for n in names), names


def test_host_only_entry_points(lib):
    L = lib.lib
    assert L.muser_cuda_abi_version() == 3
    for t, ok in [(lib.Q4_K, 1), (lib.Q5_K, 1), (lib.Q6_K, 1), (lib.NVFP4, 1), (lib.F16, 0), (8, 0), (1001, 0)]:
        assert L.muser_cuda_supports_projection(t) == ok
    # [rows/128][n_in/64][32][4][4]
    assert L.muser_cuda_nvfp4_swizzled_scale_bytes(130, 96) == 2 * 2 * 512
    assert L.muser_cuda_nvfp4_swizzled_scale_bytes(2048, 5120) == 16 * 80 * 512


def test_null_arguments_are_statuses_not_crashes(lib):
    L = lib.lib
    assert L.muser_cuda_ctx_create(0, 0, None) == 1  # BAD_ARG
    assert L.muser_cuda_weight_info_get(None, None) == 1
    assert L.muser_cuda_sync_status(None, None) == 1
    L.muser_cuda_weight_free(None)
    L.muser_cuda_ctx_destroy(None)
