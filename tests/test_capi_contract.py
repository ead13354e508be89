"""Host-only checks of the C ABI: the library loads, exports every declared
symbol, and the calls that need no GPU behave as the reference's own hosted
`capi_contract` tests expect (null handles refused, null free accepted, the
pure helpers). No kernel is launched here."""
import ctypes as C
import re
from pathlib import Path

import pytest

from tessl_b200 import build as tb
from tessl_b200 import capi

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    tb.build()
    return capi.load()


def test_every_declared_symbol_is_exported_and_bound(lib):
    header = (ROOT / "include" / "tessl_b200.h").read_text()
    declared = set(re.findall(r"TESSL_API[^;]*?\b(tessl_\w+)\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(capi.SIGNATURES), declared ^ set(capi.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None


def test_abi_version_matches_header(lib):
    header = (ROOT / "include" / "tessl_b200.h").read_text()
    v = int(re.search(r"#define TESSL_B200_ABI_VERSION (\d+)u", header).group(1))
    assert lib.tessl_abi_version() == v == capi.ABI_VERSION


def test_null_handles_are_refused_with_a_message(lib):
    err = C.create_string_buffer(256)
    assert lib.tessl_synchronize(None, err, 256) == capi.TESSL_ERR
    assert b"null runtime handle" in err.value
    out = C.c_int32(7)
    assert lib.tessl_runtime_poisoned(None, C.byref(out), err, 256) == capi.TESSL_ERR
    assert lib.tessl_runtime_set_encode_only(None, 1, err, 256) == capi.TESSL_ERR
    # err may be NULL, and a tiny buffer gets a truncated, terminated message
    assert lib.tessl_synchronize(None, None, 0) == capi.TESSL_ERR
    small = C.create_string_buffer(b"\xff" * 8, 8)
    assert lib.tessl_synchronize(None, small, 8) == capi.TESSL_ERR
    assert small.value == b"null ru"


def test_null_free_is_ok(lib):
    assert lib.tessl_runtime_free(None) == capi.TESSL_OK


def test_threadgroup_count_and_max_k(lib):
    assert lib.tessl_simd_gemv_threadgroups(0) == 0
    assert lib.tessl_simd_gemv_threadgroups(37) == 5
    # tests/gemm_q4_mlx_tensorops.rs:332-339 of the reference project
    for g in (32, 64, 128):
        mk = lib.tessl_gemm_q4_mlx_tensorops_max_k(1, 1, g)
        assert mk == (2**31 - 1) // g * g and mk + g == 2**31
    for m, n, g in ((33, 70, 64), (4096, 2, 32), (3, 100_000, 128)):
        k = lib.tessl_gemm_q4_mlx_tensorops_max_k(m, n, g)
        assert k % g == 0 and max(m, n) * k <= 2**31 - 1 < max(m, n) * (k + g)


def test_operator_on_a_null_runtime_is_refused_before_anything_else(lib):
    err = C.create_string_buffer(256)
    bank = capi.Q4MlxBank()
    st = lib.tessl_gemv_q4_mlx_simd(None, bank, capi.Buf(), capi.Buf(), capi.QuantShape(8, 64, 64), 0, None, err, 256)
    assert st == capi.TESSL_ERR and b"null runtime handle" in err.value
