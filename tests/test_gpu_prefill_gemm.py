"""GPU parity of the Q4 prefill GEMM (`gemm_q4_mlx_tensorops`) through the C ABI.

Mirrors tests/gemm_q4_mlx_tensorops.rs of the reference project: the sweep over
M in {1, 8, 33, 70}, N in {32, 64, 33, 40, 100}, K in {128, 256}, G in {32, 64, 128}
on exact (multiples of 1/64) and random activations, each output within the
derived bound gamma_t * S of the f64 product and of the small-batch kernel; a
long K; partial tiles that must not write past y; every refusal before any
launch. Then model-sized shapes against the dequant-matvec oracle within the
stated 1e-2 relative / 2e-3 absolute (after bf16 rounding).
"""
import numpy as np
import pytest

from gpu_util import SENTINEL_F32, assert_gamma_bound, assert_north_star, rt, seeded_f32, upload_bank  # noqa: F401
from oracle import api
from tessl_b200 import nn, synth

pytestmark = pytest.mark.gpu


def ref_case(m, n, k, group, random, seed_salt=0x71E5):
    """Inputs as the reference's `run_case` draws them (unit activations, scale
    0.01 + 0.04 u, bias -0.5 + 0.6 u), from one splitmix64 stream."""
    seed = seed_salt ^ (m * 1000003 + n * 4099 + k * 17 + group)
    groups = k // group
    d = synth.splitmix_draws(seed, m * k + n * k + n * groups * 2)
    x = synth.unit_from_draws(d[: m * k])
    if not random:
        x = np.round(x * np.float32(64.0)) / np.float32(64.0)
    nib = (d[m * k: m * k + n * k] % np.uint64(16)).astype(np.uint8)
    u = (synth.unit_from_draws(d[m * k + n * k:]) + np.float32(1.0)) * np.float32(0.5)
    sb = np.where(np.arange(u.size) % 2 == 0, np.float32(0.01) + np.float32(0.04) * u,
                  np.float32(-0.5) + np.float32(0.6) * u).astype(np.float32)
    return synth.f32_to_bf16_bits(x), api.q4_pack(nib), synth.f32_to_bf16_bits(sb)


def run_gemm(rt, x, packed, sb, m, n, k, group, pad=0, y_as_bf16=False):
    bank = upload_bank(rt, packed, sb)
    xb = rt.buffer_from(x)
    if y_as_bf16:
        y = rt.buffer_from(np.full(m * n + pad, 0xA5A5, np.uint16))
    else:
        y = seeded_f32(rt, m * n, pad)
    nn.gemm_q4_mlx_tensorops(rt, bank, xb, y, nn.QuantShape(n, k, group), m, y_as_bf16=y_as_bf16)
    out = y.read(np.uint16 if y_as_bf16 else np.float32, m * n + pad)
    for b in (bank.packed, bank.scales_biases, xb, y):
        b.free()
    return out


@pytest.mark.parametrize("random", [False, True])
@pytest.mark.parametrize("group", [32, 64, 128])
def test_sweep_within_the_derived_bound(rt, group, random):
    worst = 0.0
    for m in (1, 8, 33, 70):
        for n in (32, 64, 33, 40, 100):
            for k in (128, 256):
                x, packed, sb = ref_case(m, n, k, group, random)
                got = run_gemm(rt, x, packed, sb, m, n, k, group)
                assert np.all(got != SENTINEL_F32), f"unwritten output M={m} N={n} K={k} G={group}"
                worst = max(worst, assert_gamma_bound(got, packed, sb, x, m, n, k, group, extra_terms=group,
                                                      what=f"M={m} N={n} K={k} G={group}"))
                # against the small-batch kernel on the same operands
                bank, xb = upload_bank(rt, packed, sb), rt.buffer_from(x)
                simd = np.empty((m, n), np.float32)
                for r0 in range(0, m, 8):
                    mc = min(8, m - r0)
                    yc = seeded_f32(rt, mc * n)
                    nn.gemm_q4_mlx(rt, bank, xb.view(r0 * k * 2, mc * k * 2), yc, nn.QuantShape(n, k, group), mc)
                    simd[r0:r0 + mc] = yc.read(np.float32, mc * n).reshape(mc, n)
                    yc.free()
                _, mag = api.q4_affine_f64(packed, sb, x, m, n, k, group)
                bound = (api.gamma(k + 2 * (k // group) + group) + api.gamma(k + 2 * (k // group))) * mag
                assert np.all(np.abs(got.reshape(m, n).astype(np.float64) - simd) <= bound)
                for b in (bank.packed, bank.scales_biases, xb):
                    b.free()
    assert worst <= 1.0


@pytest.mark.parametrize("group", [32, 64, 128])
def test_two_cta_tiles(rt, group):
    """More than 128 rows of X: the CTA-pair kernel (256-row tiles, each CTA expanding half
    of the weight rows), with ragged last tiles in both directions."""
    for m in (129, 256, 300):
        for n in (64, 100, 257, 520):
            for k in (256, 384):
                x, packed, sb = ref_case(m, n, k, group, True, seed_salt=0x2C7A)
                got = run_gemm(rt, x, packed, sb, m, n, k, group)
                assert np.all(got != SENTINEL_F32), f"unwritten output M={m} N={n} K={k} G={group}"
                assert_gamma_bound(got, packed, sb, x, m, n, k, group, extra_terms=group,
                                   what=f"pair M={m} N={n} K={k} G={group}")


@pytest.mark.parametrize("group", [32, 64, 128])
def test_long_k(rt, group):
    m, n, k = 40, 72, 2048
    x, packed, sb = ref_case(m, n, k, group, True)
    got = run_gemm(rt, x, packed, sb, m, n, k, group)
    assert_gamma_bound(got, packed, sb, x, m, n, k, group, extra_terms=group, what=f"long K G={group}")


@pytest.mark.parametrize("group", [32, 64, 128])
def test_partial_tiles_never_write_past_y(rt, group):
    pad = 32 * 32 + 128
    for m in (1, 8, 33, 70, 129, 257):
        for n in (33, 40, 100, 257):
            x, packed, sb = ref_case(m, n, 256, group, True, seed_salt=0x9AD)
            for as_bf16 in (False, True):
                out = run_gemm(rt, x, packed, sb, m, n, 256, group, pad=pad, y_as_bf16=as_bf16)
                if as_bf16:
                    assert np.all(out[m * n:] == 0xA5A5), f"M={m} N={n} G={group}: wrote past y (bf16)"
                else:
                    assert np.all(out[m * n:] == SENTINEL_F32), f"M={m} N={n} G={group}: wrote past y"
                    assert np.all(out[: m * n] != SENTINEL_F32), f"M={m} N={n} G={group}: unwritten output"


@pytest.mark.parametrize("m,n,k,group", [(300, 520, 4096, 64), (2048, 1024, 4096, 64), (130, 12288, 1024, 128),
                                         (17, 4096, 12288, 64), (256, 384, 96, 32), (9, 151936 // 64, 4096, 64)])
def test_model_shapes_match_the_dequant_matvec(rt, m, n, k, group):
    packed, sb = synth.q4_bank(0x7E550300 + n, n, k, group)
    packed, sb = packed.view(np.uint8).reshape(-1), sb.reshape(-1)
    x = synth.normal_bf16(0x7E550307 + m, m * k)
    got = run_gemm(rt, x, packed, sb, m, n, k, group).reshape(m, n)
    want = api.q4_dense_gemm(packed, sb, x, m, n, k, group)
    assert_north_star(got, want, f"prefill {m}x{n}x{k} g{group}")
    rows = np.arange(0, m, max(1, m // 8))  # the f64 bound on a row subset (the oracle is O(MNK))
    xs = x.reshape(m, k)[rows].reshape(-1)
    assert_gamma_bound(got[rows].reshape(-1), packed, sb, xs, len(rows), n, k, group, extra_terms=group, what="subset")
    gb = run_gemm(rt, x, packed, sb, m, n, k, group, y_as_bf16=True)
    assert np.array_equal(gb, synth.f32_to_bf16_bits(got.reshape(-1)))


def _subset_rows(m):
    """Rows on either side of every 128-row boundary the tiles have, the first and the last."""
    rows = {0, m - 1}
    for b in range(128, m, 128):
        rows.update((b - 1, b))
    rows.update(range(7, m, max(1, m // 5)))
    return np.array(sorted(r for r in rows if 0 <= r < m))


def _check_rows_against_the_oracle(got, packed, sb, x, rows, n, k, group, what):
    """`rows` of the [m, n] result against the dequant-matvec (stated tolerance) and the exact product (gamma_t S)."""
    xs = np.ascontiguousarray(x.reshape(-1, k)[rows]).reshape(-1)
    want = api.q4_dense_gemm(packed, sb, xs, len(rows), n, k, group)
    assert_north_star(got[rows], want, what)
    assert_gamma_bound(got[rows].reshape(-1), packed, sb, xs, len(rows), n, k, group, extra_terms=group, what=what)


def _check_sums_against_the_oracle(got, packed, sb, x, m, n, k, group, what):
    """Every output takes part: the column sums of Y equal W (sum of the rows of X) and the row sums equal
    X (sum of the rows of W), both formed in f64 on the host from the bit-exact dequantized weights."""
    w = api.q4_dequant(packed, sb, n, k, group).astype(np.float64)
    xf = synth.bf16_bits_to_f32(x).reshape(m, k).astype(np.float64)
    g64 = got.astype(np.float64)
    col_want, row_want = w @ xf.sum(axis=0), xf @ w.sum(axis=0)
    col_tol = 1e-5 * np.abs(g64).sum(axis=0) + 1e-3
    row_tol = 1e-5 * np.abs(g64).sum(axis=1) + 1e-3
    bad = np.flatnonzero(np.abs(g64.sum(axis=0) - col_want) > col_tol)
    assert bad.size == 0, f"{what}: column sums differ at columns {bad[:8]}"
    bad = np.flatnonzero(np.abs(g64.sum(axis=1) - row_want) > row_tol)
    assert bad.size == 0, f"{what}: row sums differ at rows {bad[:8]}"


@pytest.mark.parametrize("m,n,k,group,tile", [(600, 12251, 256, 32, 256), (600, 12288, 256, 128, 256),
                                              (1024, 12288, 512, 64, 256), (300, 12288, 256, 64, 192),
                                              (300, 12200, 256, 32, 192), (2048, 12288, 256, 128, 256)])
def test_the_tile_the_library_picks_for_wide_outputs(rt, m, n, k, group, tile):
    """Shapes for which the library's own estimate picks the 256- and 192-wide tiles of the CTA-pair kernel, with
    more tiles than clusters (each cluster walks several tiles: both accumulator buffers, rings that carry on
    across tiles), ragged M and N, f32 and bf16 outputs, nothing written past y."""
    packed, sb = synth.q4_bank(0x7E550500 + n + m, n, k, group)
    packed, sb = packed.view(np.uint8).reshape(-1), sb.reshape(-1)
    x = synth.normal_bf16(0x7E550507 + m, m * k)
    pad = 4096
    out = run_gemm(rt, x, packed, sb, m, n, k, group, pad=pad)
    assert rt.last_prefill_tile() == (tile, 1), rt.last_prefill_tile()
    assert np.all(out[m * n:] == SENTINEL_F32), "wrote past y"
    got = out[: m * n].reshape(m, n)
    assert np.all(np.isfinite(got)) and np.all(got != SENTINEL_F32)
    want = api.q4_dense_gemm(packed, sb, x, m, n, k, group)
    assert_north_star(got, want, f"prefill {m}x{n}x{k} g{group} tile {tile}")
    _check_rows_against_the_oracle(got, packed, sb, x, _subset_rows(m), n, k, group, f"tile {tile} rows")
    gb = run_gemm(rt, x, packed, sb, m, n, k, group, pad=pad, y_as_bf16=True)
    assert np.array_equal(gb[: m * n], synth.f32_to_bf16_bits(got.reshape(-1)))
    assert np.all(gb[m * n:] == 0xA5A5), "wrote past y (bf16)"


def test_the_benchmarked_prefill_shape(rt):
    """BASELINE config: X [2048, 4096] bf16 ~ N(0, 1) against a 12288 x 4096 bank of group 64 - the 256-wide tile of
    the CTA-pair kernel, six tiles per cluster. Rows either side of every tile boundary against the oracle (the
    full product is 1e11 multiply-adds on the host), every output through the row and column sums, and 64 rows
    against the small-batch kernel, whose order of summation the reference's recorded vectors pin."""
    m, n, k, group = 2048, 12288, 4096, 64
    packed, sb = synth.q4_bank(0x7E550030, n, k, group)
    packed, sb = packed.view(np.uint8).reshape(-1), sb.reshape(-1)
    x = synth.normal_bf16(0x7E550031, m * k)
    out = run_gemm(rt, x, packed, sb, m, n, k, group, pad=4096)
    assert rt.last_prefill_tile() == (256, 1), rt.last_prefill_tile()
    assert np.all(out[m * n:] == SENTINEL_F32), "wrote past y"
    got = out[: m * n].reshape(m, n)
    assert np.all(np.isfinite(got)) and np.all(got != SENTINEL_F32)
    rows = _subset_rows(m)
    _check_rows_against_the_oracle(got, packed, sb, x, rows, n, k, group, "2048x12288x4096 rows")
    _check_sums_against_the_oracle(got, packed, sb, x, m, n, k, group, "2048x12288x4096")
    bank, xb = upload_bank(rt, packed, sb), rt.buffer_from(x)
    for r0 in range(0, m, 256):  # eight rows of every row tile
        yc = seeded_f32(rt, 8 * n)
        nn.gemm_q4_mlx(rt, bank, xb.view(r0 * k * 2, 8 * k * 2), yc, nn.QuantShape(n, k, group), 8)
        simd = yc.read(np.float32, 8 * n).reshape(8, n)
        yc.free()
        assert_north_star(got[r0:r0 + 8], simd, f"rows {r0}.. against the small-batch kernel")
        assert np.max(np.abs(got[r0:r0 + 8] - simd)) < 2e-3
    for b in (bank.packed, bank.scales_biases, xb):
        b.free()


@pytest.mark.parametrize("pair", [1, 0])
@pytest.mark.parametrize("tile", [128, 192, 256])
def test_every_compiled_tile_on_ragged_shapes(rt, tile, pair):
    """Each tile width of both kernels (CTA pair and single CTA), forced through the runtime's tuning hook, on
    ragged shapes: fewer tiles than clusters, and several tiles per cluster."""
    rt.set_prefill_tile(tile, pair)
    try:
        for m, n, k, group in ((300, 520, 384, 32), (129, 1000, 256, 64), (40, 72, 2048, 64), (700, 20011, 128, 128),
                               (8, 4096, 1024, 64)):
            packed, sb = synth.q4_bank(0x7E550600 + n, n, k, group)
            packed, sb = packed.view(np.uint8).reshape(-1), sb.reshape(-1)
            x = synth.normal_bf16(0x7E550607 + m, m * k)
            out = run_gemm(rt, x, packed, sb, m, n, k, group, pad=1024)
            assert rt.last_prefill_tile() == (tile, pair), rt.last_prefill_tile()
            assert np.all(out[m * n:] == SENTINEL_F32), f"tile {tile} pair {pair}: wrote past y"
            got = out[: m * n].reshape(m, n)
            assert np.all(got != SENTINEL_F32), f"tile {tile} pair {pair}: unwritten output"
            want = api.q4_dense_gemm(packed, sb, x, m, n, k, group)
            assert_north_star(got, want, f"tile {tile} pair {pair} {m}x{n}x{k} g{group}")
            rows = _subset_rows(m)[:12]
            _check_rows_against_the_oracle(got, packed, sb, x, rows, n, k, group, f"tile {tile} pair {pair}")
    finally:
        rt.set_prefill_tile(0, -1)
    with pytest.raises(nn.TesslError, match="tile_n 100"):
        rt.set_prefill_tile(100, -1)


def test_rows_of_any_magnitude_survive_the_f16_operands(rt):
    """The per-row power-of-two rescale: rows scaled by 2^-40 .. 2^+60 give the
    correspondingly scaled outputs, a zero row gives zeros."""
    m, n, k, group = 6, 64, 512, 64
    packed, sb = synth.q4_bank(77, n, k, group)
    packed, sb = packed.view(np.uint8).reshape(-1), sb.reshape(-1)
    base = synth.bf16_bits_to_f32(synth.normal_bf16(78, k))
    scales = [1.0, 2.0 ** -40, 2.0 ** 60, 2.0 ** 15, 0.0, 2.0 ** -100]
    x = np.concatenate([synth.f32_to_bf16_bits((base * np.float32(s)).astype(np.float32)) for s in scales])
    got = run_gemm(rt, x, packed, sb, m, n, k, group).reshape(m, n)
    want = api.q4_dense_gemm(packed, sb, x, m, n, k, group)
    for i, s in enumerate(scales):
        if s == 0.0:
            assert np.all(got[i] == 0.0)
        else:
            np.testing.assert_allclose(got[i] / np.float32(s), want[i] / np.float32(s), rtol=2e-3, atol=2e-3)


def test_refusals_before_any_launch(rt):
    m, n, k, g = 40, 40, 256, 64
    packed, sb = synth.q4_bank(3, n, k, g)
    bank = upload_bank(rt, packed, sb)
    x = rt.buffer_from(synth.normal_bf16(4, m * k))
    y = seeded_f32(rt, m * n)
    shape = nn.QuantShape(n, k, g)
    rt.take_dispatch_count()
    small = rt.alloc_buffer(64)
    cases = [
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, x, y, nn.QuantShape(n, k, 256), m), "group_size 256"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, x, y, nn.QuantShape(n, k, 16), m), "group_size 16"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, x, y, nn.QuantShape(n, k, 0), m), "group_size"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, x, y, nn.QuantShape(n, 250, 64), m), "multiple of group_size"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, x, y, nn.QuantShape(n, 0, 64), m), "cols must be non-zero"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, nn.Q4MlxBank(small, bank.scales_biases), x, y, shape, m), "packed"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, nn.Q4MlxBank(bank.packed, small), x, y, shape, m), "scales_biases"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, small, y, shape, m), "x_bf16"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, x, small, shape, m), " y"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, x, y, shape, 2**32 - 1), "32-bit"),
        (lambda: nn.gemm_q4_mlx_tensorops(rt, bank, x, x, shape, m), "gemm_q4_mlx_tensorops"),
    ]
    for fn, want in cases:
        with pytest.raises(nn.TesslError) as e:
            fn()
        assert want in str(e.value), (want, str(e.value))
    # the first refused K is the derived bound plus one group (tests/gemm_q4_mlx_tensorops.rs:330-371)
    for mm, nn_, gg in ((1, 1, 32), (33, 70, 64), (3, 100_000, 128)):
        max_k = nn.gemm_q4_mlx_tensorops_max_k(mm, nn_, gg)
        with pytest.raises(nn.TesslError) as e:
            nn.gemm_q4_mlx_tensorops(rt, bank, x, y, nn.QuantShape(nn_, max_k, gg), mm)
        assert "32-bit" not in str(e.value) and "gemm_q4_mlx_tensorops" in str(e.value)
        with pytest.raises(nn.TesslError, match="32-bit"):
            nn.gemm_q4_mlx_tensorops(rt, bank, x, y, nn.QuantShape(nn_, max_k + gg, gg), mm)
    nn.gemm_q4_mlx_tensorops(rt, bank, x, y, shape, 0)
    nn.gemm_q4_mlx_tensorops(rt, bank, x, y, nn.QuantShape(0, k, g), m)
    assert rt.take_dispatch_count() == 0
    assert np.all(y.read(np.float32, m * n) == SENTINEL_F32)
