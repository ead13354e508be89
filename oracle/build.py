"""Build recipe for the CPU oracle (test infrastructure; the product never imports it).

`build_oracle()` compiles `tessl_oracle.c` into `_build/libtessl_oracle.so`.
`build_ref(ref_root)` compiles the reference's own kernel sources, where they
lie under the reference checkout (the argument or $TESSL_REFERENCE_ROOT), into
`_ref/libtessl_ref_kernels.so` (see `ref_shim/`); without a checkout it returns
the library built earlier, or None.
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


def _kernel_blocks(text: str, names: list[str]) -> str:
    """The `kernel void NAME(...) { ... }` definitions of `names`, cut out of a Metal source by brace matching."""
    import re

    out = []
    for name in names:
        m = re.search(r"kernel\s+void\s+" + re.escape(name) + r"\s*\(", text)
        if not m:
            raise RuntimeError(f"reference kernel source no longer defines {name}")
        i = text.index("{", m.end())
        depth, j = 0, i
        while True:
            depth += {"{": 1, "}": -1}.get(text[j], 0)
            j += 1
            if depth == 0:
                break
        out.append(text[m.start():j])
    return "\n\n".join(out) + "\n"


def reference_root(ref_root: str | os.PathLike | None = None) -> Path | None:
    """The reference checkout: the argument, else $TESSL_REFERENCE_ROOT, else a folder named `reference`
    beside this repository; None if none of them holds the kernel sources."""
    candidates = [ref_root, os.environ.get("TESSL_REFERENCE_ROOT"), HERE.parent.parent / "reference"]
    for root in candidates:
        if root and (Path(root) / "kernels" / "gemv_q8.metal").exists():
            return Path(root)
    return None


def build_ref(ref_root: str | os.PathLike | None = None, force: bool = False) -> Path | None:
    """Compile the reference's Q4/Q8 simdgroup kernel sources as C++ against `ref_shim/`.

    The sources are read where they lie in the reference checkout (`ref_root`, else
    $TESSL_REFERENCE_ROOT): `[[attribute]]` annotations are dropped (C++ has no meaning for buffer
    slots; the harness passes arguments in declaration order), the row-major `gemv_q4_mlx_simd*` and
    `gemm_q4_mlx_simd*` entry points are cut out of their files, and the result goes to a temporary
    folder that is deleted after the compile: no reference source is copied into this repository, only
    the shared object lands in `_ref/`. Without a checkout this returns the existing `_ref` library,
    or None.
    """
    import re

    ref = reference_root(ref_root)
    if ref is None:
        return REF_SO if REF_SO.exists() else None
    kernels = ref / "kernels"
    shim = HERE / "ref_shim"
    deps = ["gemv_q4_mlx.metal", "gemm_q4_mlx.metal", "gemv_q8.metal", "gemv_q4_mlx_simd.h", "gemm_q4_mlx_simd.h",
            "q4_mlx_dot.h", "act.h"]
    sources = [shim / "harness.cpp", shim / "metal_stdlib", *[kernels / k for k in deps]]
    if not force and not _stale(REF_SO, sources):
        return REF_SO

    def strip(text: str) -> str:
        return re.sub(r"\[\[[^\]]*\]\]", "", text)

    with tempfile.TemporaryDirectory(prefix="tessl_ref_") as tmp:
        t = Path(tmp)
        (t / "gemv_q8.inc").write_text(strip((kernels / "gemv_q8.metal").read_text()))
        (t / "gemm_q4_mlx_entries.inc").write_text(
            strip(_kernel_blocks((kernels / "gemm_q4_mlx.metal").read_text(), ["gemm_q4_mlx_simd", "gemm_q4_mlx_simd_add"])))
        (t / "gemv_q4_mlx_simd_entries.inc").write_text(
            strip(_kernel_blocks((kernels / "gemv_q4_mlx.metal").read_text(),
                                 ["gemv_q4_mlx_simd", "gemv_q4_mlx_simd_add", "gemv_q4_mlx_simd_gate_up_gelu",
                                  "gemv_q4_mlx_simd_gate_up_silu", "gemv_q4_mlx_simd_kv", "gemv_q4_mlx_simd_qkv"])))
        for h in ("gemv_q4_mlx_simd.h", "gemm_q4_mlx_simd.h", "q4_mlx_dot.h", "act.h"):
            (t / h).write_text(strip((kernels / h).read_text()))
        _compile(
            [str(shim / "harness.cpp")],
            REF_SO,
            cxx=True,
            extra=["-std=c++20", "-pthread", "-fno-strict-aliasing", "-Wno-unused-parameter", "-Wno-unused-variable",
                   "-Wno-sign-compare", "-Wno-unknown-pragmas", "-Wno-unused-function", "-I", str(shim), "-I", tmp],
        )
    return REF_SO


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None, help="reference checkout (else $TESSL_REFERENCE_ROOT): also build _ref/ from it")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(force=a.force))
    if reference_root(a.ref):
        print(build_ref(a.ref, force=a.force))
    sys.exit(0)
