"""Builds libmuser_cuda.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libmuser_cuda.so"
SOURCES = ["api.cu", "repack.cu", "kquant_decode.cu", "kquant_tc.cu", "nvfp4_quant.cu", "nvfp4_gemm.cu", "nvfp4_static.cu", "nvfp4_a16.cu", "collective.cu", "layer_ops.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    return os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _newest(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def build(force: bool = False, verbose: bool = False) -> Path:
    srcs = [CSRC / s for s in SOURCES]
    deps = list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "muser_cuda.h"]
    if not force and LIB.exists() and LIB.stat().st_mtime >= _newest(srcs + deps):
        return LIB
    objdir = CSRC / "build"
    objdir.mkdir(exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime >= _newest([src] + deps):
            return obj
        extra = os.environ.get("MUSER_CUDA_NVCC_EXTRA", "").split()  # e.g. -DMUSER_GEMM_WAIT_PROFILE for a development build
        cmd = [nvcc(), *NVCC_FLAGS, *extra, "-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (objdir / (src.stem + ".ptxas.log")).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr[-4000:]}")
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xlinker", "--version-script=" + str(CSRC / "exports.map"), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
