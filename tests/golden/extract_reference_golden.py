"""Extracts the reference's recorded known-answer table for the Q4 kernels.

Reads `tests/q4_kernels_template.rs` of a reference checkout as text, parses
its `GOLDEN` table (kernel entry, case, FNV-1a hash of every output word, first
eight output words) and writes the rows that pin the path built here to
`q4_kernels_golden.json` beside this script. The rows were recorded by the
reference's author from the kernels running on an Apple GPU.

    python tests/golden/extract_reference_golden.py /path/to/reference      (or TESSL_REFERENCE_ROOT=...)
"""
import json
import re
import sys
from pathlib import Path

KEEP = {
    # row-major simdgroup GEMV / small-M GEMM entries (the hot path)
    "gemv_q4_mlx_simd", "gemv_q4_mlx_simd_add", "gemv_q4_mlx_simd_gate_up_gelu", "gemv_q4_mlx_simd_kv",
    "gemv_q4_mlx_simd_qkv", "gemm_q4_mlx_simd", "gemm_q4_mlx_simd_add",
    # the f32 -> bf16 device cast rule the bf16 outputs follow
    "cast_f32_to_bf16", "cast_bf16_to_f32",
}


def main() -> None:
    import os

    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TESSL_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: extract_reference_golden.py <reference checkout>   (or set TESSL_REFERENCE_ROOT)")
    ref = Path(root)
    text = (ref / "tests" / "q4_kernels_template.rs").read_text()
    body = text[text.index("const GOLDEN: &[Golden] = &["):]
    body = body[: body.index("\n];")]
    row = re.compile(r'\(\s*"([^"]+)",\s*"([^"]+)",\s*(0x[0-9a-f]+),\s*\[\s*([^\]]+?)\s*\],?\s*\)', re.S)
    rows = []
    for kernel, case, h, words in row.findall(body):
        if kernel not in KEEP:
            continue
        ws = [int(w, 16) for w in re.findall(r"0x[0-9a-f]+", words)]
        assert len(ws) == 8, (kernel, case)
        rows.append({"kernel": kernel, "case": case, "hash": h, "first_words": [f"{w:#010x}" for w in ws]})
    # The f32 edge-case bit patterns the cast rows start their input with.
    sp = text[text.index("const F32_SPECIALS: &[u32] = &["):]
    sp = sp[: sp.index("];")]
    specials = [f"{int(w.replace('_', ''), 16):#010x}" for w in re.findall(r"0x[0-9a-f_]+", sp)]
    out = Path(__file__).with_name("q4_kernels_golden.json")
    out.write_text(json.dumps({"source": "tests/q4_kernels_template.rs GOLDEN and F32_SPECIALS (reference project path)",
                               "f32_specials": specials, "rows": rows}, indent=1) + "\n")
    print(f"{len(rows)} rows -> {out}")


if __name__ == "__main__":
    main()
