// Runs the reference project's MLX-Q4 / Q8 simdgroup kernels, compiled from its own sources against
// the stand-in metal_stdlib of this folder, over the grid its Rust host dispatches
// (src/nn.rs: ceil(rows / 8) threadgroups of 2 simdgroups x 32 lanes; K/V and Q/K/V launches
// partition the grid by bank). Test infrastructure: the CPU oracle is checked against this.
//
// The `.inc` files are produced at build time from the reference checkout (attributes stripped;
// for gemv_q4_mlx.metal only the `gemv_q4_mlx_simd*` row-major entry points are cut out) and are
// never stored in this repository.
#include <thread>
#include <vector>

using os_thread = std::thread;  // named before the stand-in header defines Metal's `thread` qualifier away

#include <metal_stdlib>

#include "gemv_q4_mlx_simd.h"
#include "gemm_q4_mlx_simd.h"
#include "gemv_q8.inc"
#include "gemm_q4_mlx_entries.inc"
#include "gemv_q4_mlx_simd_entries.inc"

namespace {

/// `fn(tgid, sgid, lane)` for every thread of `tgs` threadgroups, one simdgroup (32 threads) at a time.
template <typename F>
void run_grid(unsigned tgs, unsigned sg_per_tg, F fn)
{
    for (unsigned tg = 0; tg < tgs; ++tg) {
        for (unsigned sg = 0; sg < sg_per_tg; ++sg) {
            metal::emu::Simdgroup group;
            std::vector<os_thread> lanes;
            lanes.reserve(32);
            for (unsigned l = 0; l < 32; ++l) {
                lanes.emplace_back([&, l] {
                    metal::emu::group = &group;
                    metal::emu::lane = l;
                    fn(tg, sg, l);
                    // a lane that left before a simd_sum (row0 >= rows) must not leave the others waiting
                    group.bar.arrive_and_drop();
                });
            }
            for (auto &t : lanes) t.join();
        }
    }
}

unsigned tgs_for(unsigned rows) { return (rows + 7u) / 8u; }

}  // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API void ref_gemv_q8(const signed char *packed, const float *scales, const float *zeros, const float *x, float *y,
                         unsigned rows, unsigned cols, unsigned group_size)
{
    run_grid(tgs_for(rows), 2, [&](unsigned tg, unsigned sg, unsigned lane) {
        gemv_q8(reinterpret_cast<const char *>(packed), scales, zeros, x, y, rows, cols, group_size, tg, sg, lane);
    });
}

REF_API void ref_gemv_q4_mlx_simd(const uchar *packed, const uint16_t *sb, const uint16_t *x, float *y, unsigned rows,
                                  unsigned cols, unsigned group_size, const float *resid)
{
    const auto *sbp = reinterpret_cast<const metal::bfloat2 *>(sb);
    const auto *xp = reinterpret_cast<const metal::bfloat *>(x);
    run_grid(tgs_for(rows), 2, [&](unsigned tg, unsigned sg, unsigned lane) {
        if (resid) {
            gemv_q4_mlx_simd_add(packed, sbp, nullptr, xp, y, rows, cols, group_size, resid, tg, sg, lane);
        } else {
            gemv_q4_mlx_simd(packed, sbp, nullptr, xp, y, rows, cols, group_size, tg, sg, lane);
        }
    });
}

REF_API void ref_gemv_q4_mlx_simd_gate_up(const uchar *gate, const uint16_t *gate_sb, const uchar *up, const uint16_t *up_sb,
                                          const uint16_t *x, float *mid, unsigned rows, unsigned cols, unsigned group_size,
                                          unsigned mid_as_bf16, int silu)
{
    const auto *gs = reinterpret_cast<const metal::bfloat2 *>(gate_sb), *us = reinterpret_cast<const metal::bfloat2 *>(up_sb);
    const auto *xp = reinterpret_cast<const metal::bfloat *>(x);
    run_grid(tgs_for(rows), 2, [&](unsigned tg, unsigned sg, unsigned lane) {
        if (silu) {
            gemv_q4_mlx_simd_gate_up_silu(gate, gs, nullptr, up, us, nullptr, xp, mid, rows, cols, group_size, mid_as_bf16, tg, sg,
                                          lane);
        } else {
            gemv_q4_mlx_simd_gate_up_gelu(gate, gs, nullptr, up, us, nullptr, xp, mid, rows, cols, group_size, mid_as_bf16, tg, sg,
                                          lane);
        }
    });
}

REF_API void ref_gemv_q4_mlx_simd_kv(const uchar *k, const uint16_t *k_sb, const uchar *v, const uint16_t *v_sb,
                                     const uint16_t *x, float *k_out, float *v_out, unsigned rows, unsigned cols,
                                     unsigned group_size)
{
    const unsigned tg_k = tgs_for(rows);
    const auto *ks = reinterpret_cast<const metal::bfloat2 *>(k_sb), *vs = reinterpret_cast<const metal::bfloat2 *>(v_sb);
    const auto *xp = reinterpret_cast<const metal::bfloat *>(x);
    run_grid(2 * tg_k, 2, [&](unsigned tg, unsigned sg, unsigned lane) {
        gemv_q4_mlx_simd_kv(k, ks, nullptr, v, vs, nullptr, xp, k_out, v_out, rows, cols, group_size, tg_k, tg, sg, lane);
    });
}

REF_API void ref_gemv_q4_mlx_simd_qkv(const uchar *q, const uint16_t *q_sb, const uchar *k, const uint16_t *k_sb, const uchar *v,
                                      const uint16_t *v_sb, const uint16_t *x, float *q_out, float *k_out, float *v_out,
                                      unsigned rows_q, unsigned rows_kv, unsigned cols, unsigned group_size)
{
    const unsigned tg_q = tgs_for(rows_q), tg_k = tgs_for(rows_kv);
    const auto *qs = reinterpret_cast<const metal::bfloat2 *>(q_sb), *ks = reinterpret_cast<const metal::bfloat2 *>(k_sb),
               *vs = reinterpret_cast<const metal::bfloat2 *>(v_sb);
    const auto *xp = reinterpret_cast<const metal::bfloat *>(x);
    run_grid(tg_q + 2 * tg_k, 2, [&](unsigned tg, unsigned sg, unsigned lane) {
        gemv_q4_mlx_simd_qkv(q, qs, k, ks, v, vs, xp, q_out, k_out, v_out, rows_q, rows_kv, cols, group_size, tg_q, tg_k, tg, sg,
                             lane);
    });
}

REF_API void ref_gemm_q4_mlx_simd(const uchar *packed, const uint16_t *sb, const uint16_t *x, float *y, unsigned rows,
                                  unsigned cols, unsigned group_size, unsigned m, const float *resid)
{
    const auto *sbp = reinterpret_cast<const metal::bfloat2 *>(sb);
    const auto *xp = reinterpret_cast<const metal::bfloat *>(x);
    run_grid(tgs_for(rows), 2, [&](unsigned tg, unsigned sg, unsigned lane) {
        if (resid) {
            gemm_q4_mlx_simd_add(packed, sbp, nullptr, xp, y, rows, cols, group_size, m, resid, tg, sg, lane);
        } else {
            gemm_q4_mlx_simd(packed, sbp, nullptr, xp, y, rows, cols, group_size, m, tg, sg, lane);
        }
    });
}
