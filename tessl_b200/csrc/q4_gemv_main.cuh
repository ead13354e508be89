// The kernel body that goes with q4_gemv_kernel.cuh: persistent blocks, split K
// across warps, double-buffered weight loads.
#pragma once

#include "q4_gemv_kernel.cuh"

namespace tessl {
namespace q4k {

/// One warp's loads for one row group: R rows x NCH chunks x NB banks.
template <int NB, int R, int NCH>
struct Unit {
    uint4 wq[R][NCH][NB];
    uint32_t sbw[R][NCH][NB];
};

struct Where {
    Seg sg;
    uint32_t row0;
};

__device__ __forceinline__ Where locate(const Params &p, uint32_t g, int rows_per_group)
{
    int s = 0;
    if (p.nseg > 1 && g >= p.seg[1].group_begin) s = 1;
    if (p.nseg > 2 && g >= p.seg[2].group_begin) s = 2;
    Where w;
    w.sg = p.seg[s];
    w.row0 = (g - w.sg.group_begin) * rows_per_group;
    return w;
}

/// M activation rows, NB banks (2 = gate/up), R rows per group, NCH chunks per
/// warp held in registers (x stays resident). NCH == 0 selects the streaming
/// form for very long rows and for M > 1: one chunk at a time, x re-read from
/// cache for every unit.
template <int M, int NB, int R, int NCH>
__global__ void __launch_bounds__(256) q4_gemv_kernel(const Params p)
{
    constexpr int NC = NCH == 0 ? 1 : NCH;  // chunks per unit
    constexpr int V = R * NB * M;           // accumulators per lane
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const uint32_t cols = p.cols;
    const uint32_t gpr = cols >> p.group_shift;
    const size_t row_bytes = cols >> 1;
    const uint32_t nchunks = (cols + kChunk - 1) / kChunk;
    // Streaming form: this warp's chunks are warp, warp + W, ...; resident form: exactly NCH of them.
    const uint32_t my_chunks = NCH == 0 ? (nchunks > (uint32_t)warp ? (nchunks - warp + nwarps - 1) / nwarps : 0) : NCH;

    __shared__ float red[2][8][V < 32 ? 32 : V];

    // Resident activations.
    uint32_t xr[NC][M][16];
    float xs[NC][M];
    if constexpr (NCH != 0) {
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const uint32_t k0 = (warp + c * nwarps) * kChunk + lane * 32;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                load_x32(p.x, (size_t)m * cols + k0, k0 < cols, xr[c][m]);
                xs[c][m] = xsum32(xr[c][m]);
            }
        }
    }

    // Per-lane constants of the resident form: which of the warp's chunks this
    // lane has columns in, and the byte / group offsets of its slice.
    bool live_c[NC];
    uint32_t koff[NC], goff[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const uint32_t k0 = (warp + c * nwarps) * kChunk + lane * 32;
        live_c[c] = k0 < cols;
        koff[c] = k0 >> 1;
        goff[c] = k0 >> p.group_shift;
    }

    // `full`: all R rows of the group exist (only a bank's last group can be short;
    // its missing rows re-read the last row and their sums are never stored).
    auto load_unit = [&](Unit<NB, R, NC> &u, const Where &w, uint32_t chunk_base) {
        const bool full = w.row0 + R <= w.sg.rows;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            bool live;
            uint32_t ko, go;
            if constexpr (NCH == 0) {
                const uint32_t k0 = (chunk_base + c * nwarps) * kChunk + lane * 32;
                live = k0 < cols, ko = k0 >> 1, go = k0 >> p.group_shift;
            } else {
                live = live_c[c], ko = koff[c], go = goff[c];
            }
            if (!live) continue;  // the buffers were zeroed once; a dead lane never overwrites them
            const uint8_t *pk0 = w.sg.packed0 + (size_t)w.row0 * row_bytes + ko;
            const uint32_t *sb0 = w.sg.sb0 + (size_t)w.row0 * gpr + go;
            const uint8_t *pk1 = NB == 2 ? w.sg.packed1 + (size_t)w.row0 * row_bytes + ko : nullptr;
            const uint32_t *sb1 = NB == 2 ? w.sg.sb1 + (size_t)w.row0 * gpr + go : nullptr;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t rr = full ? (uint32_t)r : min((uint32_t)r, w.sg.rows - 1 - w.row0);
                u.wq[r][c][0] = dev::ldg_stream16(pk0 + rr * row_bytes);
                u.sbw[r][c][0] = dev::ldg_stream4(sb0 + (size_t)rr * gpr);
                if constexpr (NB == 2) {
                    u.wq[r][c][1] = dev::ldg_stream16(pk1 + rr * row_bytes);
                    u.sbw[r][c][1] = dev::ldg_stream4(sb1 + (size_t)rr * gpr);
                }
            }
        }
    };

    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.0f;

    auto compute_unit = [&](const Unit<NB, R, NC> &u, uint32_t chunk_base) {
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            if constexpr (NCH == 0) {
                const uint32_t k0 = (chunk_base + c * nwarps) * kChunk + lane * 32;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    load_x32(p.x, (size_t)m * cols + k0, k0 < cols, xr[c][m]);
                    xs[c][m] = xsum32(xr[c][m]);
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const float scale = dev::bf16_lo(u.sbw[r][c][b]), bias = dev::bf16_hi(u.sbw[r][c][b]);
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const float dot = fmaf(-128.0f, xs[c][m], dot32_biased(u.wq[r][c][b], xr[c][m]));
                        float &a = acc[(r * NB + b) * M + m];
                        a = fmaf(scale, dot, fmaf(bias, xs[c][m], a));
                    }
                }
            }
        }
    };

    int buf = 0;
    auto finish_group = [&](const Where &w) {
        // Lanes, then warps (fixed order), then the epilogue: one thread per output.
        if constexpr (V == 1 || V == 2 || V == 4 || V == 8 || V == 16 || V == 32) {
            transpose_reduce<V>(acc, lane);
            if ((lane & (32 / V - 1)) == 0) red[buf][warp][owned_index<V>(lane)] = acc[0];
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float t = dev::warp_sum(acc[i]);
                if (lane == 0) red[buf][warp][i] = t;
            }
        }
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.0f;
        __syncthreads();
        const int t = threadIdx.x;
        if (t < R * M) {
            const int r = t / M, m = t % M;
            const uint32_t row = w.row0 + r;
            if (row < w.sg.rows) {
                float sum[NB];
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    float v = red[buf][0][(r * NB + b) * M + m];
                    for (int ww = 1; ww < nwarps; ++ww) v += red[buf][ww][(r * NB + b) * M + m];
                    sum[b] = v;
                }
                const size_t idx = (size_t)m * w.sg.rows + row;
                float v = sum[0];
                if (p.epi == EPI_ADD_RESID) {
                    v = v + w.sg.resid[idx];
                } else if (p.epi == EPI_GATE_UP_SILU) {
                    v = dev::silu(sum[0]) * sum[NB - 1];
                } else if (p.epi == EPI_GATE_UP_GELU) {
                    v = dev::gelu_pytorch_tanh(sum[0]) * sum[NB - 1];
                }
                if (p.out_bf16) {
                    static_cast<uint16_t *>(w.sg.out)[idx] = dev::f32_to_bf16_store(v);
                } else {
                    static_cast<float *>(w.sg.out)[idx] = v;
                }
            }
        }
        buf ^= 1;
    };

    // Units in program order: for each of the block's groups, this warp's chunk
    // steps. Resident form: one unit per group. Streaming form: my_chunks units.
    const uint32_t steps = NCH == 0 ? my_chunks : 1;
    uint32_t g = blockIdx.x, step = 0;
    if (g >= p.ngroups) return;
    Unit<NB, R, NC> ua, ub;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                ua.wq[r][c][b] = ub.wq[r][c][b] = make_uint4(0, 0, 0, 0);
                ua.sbw[r][c][b] = ub.sbw[r][c][b] = 0;
            }
    Where wa = locate(p, g, R), wb = wa;
    uint32_t ca = warp, cb = warp;  // chunk base of the unit in each buffer
    bool have_a = true, have_b = false;
    if (steps > 0) load_unit(ua, wa, ca);

    // advance (g, step) to the next unit; returns false at the end
    auto next = [&](uint32_t &gg, uint32_t &st) {
        if (st + 1 < steps) {
            ++st;
            return true;
        }
        st = 0;
        gg += gridDim.x;
        return gg < p.ngroups;
    };

    while (true) {
        // ---- buffer A holds (g, step); prefetch its successor into B
        uint32_t g2 = g, s2 = step;
        have_b = next(g2, s2);
        if (have_b) {
            if (g2 != g) wb = locate(p, g2, R);
            else wb = wa;
            cb = warp + s2 * nwarps;
            if (steps > 0) load_unit(ub, wb, cb);
        }
        if (steps > 0) compute_unit(ua, ca);
        if (step + 1 >= steps) finish_group(wa);
        if (!have_b) break;
        g = g2, step = s2;
        // ---- buffer B holds (g, step); prefetch its successor into A
        g2 = g, s2 = step;
        have_a = next(g2, s2);
        if (have_a) {
            if (g2 != g) wa = locate(p, g2, R);
            else wa = wb;
            ca = warp + s2 * nwarps;
            if (steps > 0) load_unit(ua, wa, ca);
        }
        if (steps > 0) compute_unit(ub, cb);
        if (step + 1 >= steps) finish_group(wb);
        if (!have_a) break;
        g = g2, step = s2;
    }
}

}  // namespace q4k
}  // namespace tessl
