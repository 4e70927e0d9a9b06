"""Builds libbitnet_cuda_kernels.so from csrc/ with nvcc for sm_100a, in-tree.

Usage: ``python -m bitnet_mlx_rs_b200.build [--force] [--verbose]``.  nvcc cross-compiles
without a GPU, so this runs anywhere the CUDA toolkit is installed.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libbitnet_cuda_kernels.so"
SOURCES = ["abi.cu", "backend.cu", "quant_kernels.cu", "generic_gemm.cu", "decode_gemv.cu", "decode_group.cu", "prefill_gemm.cu", "midm_gemm.cu", "noalloc.cu", "decoder_kernels.cu", "decoder.cu", "weights_kernels.cu", "collective.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    # exact fp32 in the quantiser: no fast-math, no fused multiply-add across its operations
    "--fmad=false", "--prec-div=true", "--prec-sqrt=true", "--ftz=false",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libbitnet_cuda_kernels")
    return cand


def _sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list((PKG.parent / "include").glob("*.h")) + [Path(__file__)]
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a bare compiler driver; nvcc must use the system g++
    extra = ["-ccbin", shutil.which("g++") or "g++"]

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            r = subprocess.run(cmd, capture_output=True, text=True, env=env)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    if force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", *extra, "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB),
               *map(str, objs), "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libbitnet_cuda_kernels.so failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
