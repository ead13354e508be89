"""Build recipe for the CPU oracle (test infrastructure; the product never imports it).

`build_oracle()` compiles `tessl_oracle.c` into `_build/libtessl_oracle.so`.
`build_ref(ref_root)` compiles the reference's own kernel sources, where they
lie under the reference checkout, into `_ref/libtessl_ref_kernels.so` (see
`ref_shim/`); it is a no-op returning None where the checkout is absent.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "_build" / "libtessl_oracle.so"
REF_SO = HERE / "_ref" / "libtessl_ref_kernels.so"

_CFLAGS = ["-O2", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-fvisibility=hidden", "-Wall", "-Wextra"]


def _compilers(cxx: bool) -> list[str]:
    names = ["/usr/bin/g++", "g++", "c++"] if cxx else ["/usr/bin/gcc", "gcc", "cc"]
    return [n for n in names if shutil.which(n)]


def _compile(sources: list[str], out: Path, cxx: bool, extra: list[str]) -> None:
    out.parent.mkdir(parents=True, exist_ok=True)
    errors = []
    # OpenMP first (the multi-core CPU baseline wants it); some compiler drivers
    # in the image lack libgomp, so fall back to a serial build rather than fail.
    for omp in (["-fopenmp"], []):
        for cc in _compilers(cxx):
            cmd = [cc, *omp, *_CFLAGS, *extra, "-o", str(out), *sources, "-lm"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return
            errors.append(f"$ {' '.join(cmd)}\n{r.stderr}")
    raise RuntimeError("oracle build failed:\n" + "\n".join(errors))


def _stale(out: Path, sources: list[Path]) -> bool:
    return not out.exists() or any(s.stat().st_mtime > out.stat().st_mtime for s in sources)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "tessl_oracle.c"
    if force or _stale(ORACLE_SO, [src]):
        _compile([str(src)], ORACLE_SO, cxx=False, extra=[])
    return ORACLE_SO


def build_ref(ref_root: str | os.PathLike = "/root/reference", force: bool = False) -> Path | None:
    """Compile the reference's Q4/Q8 kernel sources as C++ against `ref_shim/`.

    The `.metal` files are read from the reference checkout, their
    `[[attribute]]` annotations are dropped (C++ has no meaning for buffer
    slots; the harness passes arguments in declaration order) and the result
    is written to a temporary folder that is deleted after the compile: no
    reference source is copied into this repository, only the shared object
    lands in `_ref/`.
    """
    import re

    ref = Path(ref_root)
    kernels = ref / "kernels"
    wanted = ["gemv_q4_mlx.metal", "gemm_q4_mlx.metal", "gemv_q8.metal"]
    if not all((kernels / k).exists() for k in wanted):
        return REF_SO if REF_SO.exists() else None
    shim = HERE / "ref_shim"
    sources = [shim / "harness.cpp", shim / "metal_stdlib", *[kernels / k for k in wanted]]
    if not force and not _stale(REF_SO, sources):
        return REF_SO
    with tempfile.TemporaryDirectory(prefix="tessl_ref_") as tmp:
        for k in wanted:
            text = (kernels / k).read_text()
            text = re.sub(r"\[\[[^\]]*\]\]", "", text)
            (Path(tmp) / (Path(k).stem + ".inc")).write_text(text)
        _compile(
            [str(shim / "harness.cpp")],
            REF_SO,
            cxx=True,
            extra=["-std=c++20", "-fno-strict-aliasing", "-Wno-unused-parameter", "-Wno-unused-variable",
                   "-Wno-sign-compare", "-Wno-unknown-pragmas", "-I", str(shim), "-I", str(kernels), "-I", tmp],
        )
    return REF_SO


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None, help="reference checkout; also build _ref/ from it")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(force=a.force))
    if a.ref:
        print(build_ref(a.ref, force=a.force))
    sys.exit(0)
