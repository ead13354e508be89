"""Builds the CUDA library in-tree: `tessl_b200/_lib/libtessl_b200.so`.

One `nvcc` invocation for sm_100a (the only target this library has). nvcc
cross-compiles without a GPU, so this also runs on a CPU-only build box.

    python -m tessl_b200.build [--force] [--verbose-ptxas]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "_lib" / "libtessl_b200.so"
STEP_DRIVER = HERE / "_lib" / "tessl_step_driver"
SOURCES = ["capi.cu", "nn_q4.cu", "nn_q8.cu", "q4_weight.cu", "prefill_gemm.cu", "peer_gather.cu", "qwen35_norm.cu", "mlx_q4_loader.cu"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or add it to PATH)")


def is_stale() -> bool:
    if not LIB.exists() or not STEP_DRIVER.exists():
        return True
    t = min(LIB.stat().st_mtime, STEP_DRIVER.stat().st_mtime)
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cpp"))
    deps.append(HERE.parent / "include" / "tessl_b200.h")
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose_ptxas: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    LIB.parent.mkdir(parents=True, exist_ok=True)
    host_cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else None
    cmd = [nvcc_path(), "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
           "-Xlinker", "--exclude-libs,ALL"]
    if host_cxx:
        cmd += ["-ccbin", host_cxx]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("TESSL_B200_NVCC_FLAGS", "").split()
    cmd += ["-o", str(LIB)] + [str(CSRC / s) for s in SOURCES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n$ " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if verbose_ptxas:
        sys.stderr.write(r.stderr)
    build_step_driver(host_cxx)
    return LIB


def build_step_driver(host_cxx=None) -> Path:
    """The compiled host of the end-to-end measurement (csrc/host_step_driver.cpp): plain C++ over the
    public header, linked against the library beside it (found at run time through $ORIGIN)."""
    cmd = [nvcc_path(), "-std=c++17", "-O2", "-o", str(STEP_DRIVER), str(CSRC / "host_step_driver.cpp"),
           "-L", str(LIB.parent), "-ltessl_b200", "-Xlinker", "-rpath,$ORIGIN", "-Xcompiler", "-pthread"]
    if host_cxx:
        cmd += ["-ccbin", host_cxx]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("step driver build failed:\n$ " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return STEP_DRIVER


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose-ptxas", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose_ptxas=a.verbose_ptxas))
