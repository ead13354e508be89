// Q4 GEMV (M = 1) for rows of at most 4096 columns: one warp per block, no
// shared memory, no barriers.
//
// Every decode projection whose input is the hidden state (q/k/v, o, gate/up,
// LM head at hidden 4096) has a packed row of at most 2 KiB, so one warp can keep
// the WHOLE activation vector resident (NCH <= 4 chunks x 16 packed registers)
// and own complete rows. That removes the cross-warp reduction of the split-K
// kernel (q4_gemv_main.cuh), whose per-group __syncthreads showed up as the
// second largest stall. Work is cut per warp on the host: each block gets the
// same number of consecutive rows (a multiple of R) and the grid fits the SMs
// in one wave, so the hardware block scheduler balances it.
//
// Launch overlap: the kernel is launched with programmatic stream
// serialization. It first lets its own dependents launch, prefetches the start
// of its weight rows into L2 (weights are never produced by the preceding
// kernel; a prefetch is harmless even if they were), and only then waits for
// the preceding kernel before it reads x or writes y. Back-to-back projections
// of one token therefore overlap their ramp and drain.
#pragma once

#include "q4_gemv_kernel.cuh"

namespace tessl {
namespace q4k {

struct WarpSeg {
    const uint8_t *packed0;
    const uint32_t *sb0;
    const uint8_t *packed1;
    const uint32_t *sb1;
    void *out;
    const float *resid;
    uint32_t rows;
    uint32_t block_begin;  // first block of this bank within the grid
};

struct WarpParams {
    WarpSeg seg[3];
    int nseg;
    uint32_t rows_per_block;
    const uint16_t *x;
    uint32_t cols;
    uint32_t group_shift;
    int epi;
    int out_bf16;
};

template <int NB, int R, int NCH>
struct WarpUnit {
    uint4 wq[R][NCH][NB];
    uint32_t sbw[R][NCH][NB];
};

template <int NB, int R, int NCH>
__global__ void __launch_bounds__(32, 12) q4_gemv_warp_kernel(const WarpParams p)
{
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x;
    int s = 0;
    if (p.nseg > 1 && blockIdx.x >= p.seg[1].block_begin) s = 1;
    if (p.nseg > 2 && blockIdx.x >= p.seg[2].block_begin) s = 2;
    const WarpSeg sg = p.seg[s];
    const uint32_t cols = p.cols;
    const uint32_t gpr = cols >> p.group_shift;
    const size_t row_bytes = cols >> 1;
    const uint32_t row_begin = (blockIdx.x - sg.block_begin) * p.rows_per_block;
    const uint32_t row_end = min(row_begin + p.rows_per_block, sg.rows);

    // Pull the head of this warp's rows towards L2 while the previous kernel drains.
    if (lane < NB) {
        const uint8_t *base = (lane == 0 ? sg.packed0 : sg.packed1) + (size_t)row_begin * row_bytes;
        uint32_t bytes = (uint32_t)min((size_t)(row_end - row_begin) * row_bytes, (size_t)16384);
        bytes &= ~15u;
        if (bytes) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base), "r"(bytes) : "memory");
    }

    bool live[NCH];
    uint32_t koff[NCH], goff[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const uint32_t k0 = c * kChunk + lane * 32;
        live[c] = k0 < cols;
        koff[c] = k0 >> 1;
        goff[c] = k0 >> p.group_shift;
    }

    WarpUnit<NB, R, NCH> ua, ub;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                ua.wq[r][c][b] = ub.wq[r][c][b] = make_uint4(0, 0, 0, 0);
                ua.sbw[r][c][b] = ub.sbw[r][c][b] = 0;
            }

    auto load_unit = [&](WarpUnit<NB, R, NCH> &u, uint32_t row0) {
        const bool full = row0 + R <= sg.rows;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            if (!live[c]) continue;
            const uint8_t *pk0 = sg.packed0 + (size_t)row0 * row_bytes + koff[c];
            const uint32_t *sb0 = sg.sb0 + (size_t)row0 * gpr + goff[c];
            const uint8_t *pk1 = NB == 2 ? sg.packed1 + (size_t)row0 * row_bytes + koff[c] : nullptr;
            const uint32_t *sb1 = NB == 2 ? sg.sb1 + (size_t)row0 * gpr + goff[c] : nullptr;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t rr = full ? (uint32_t)r : min((uint32_t)r, sg.rows - 1 - row0);
                u.wq[r][c][0] = dev::ldg_stream16(pk0 + rr * row_bytes);
                u.sbw[r][c][0] = dev::ldg_stream4(sb0 + (size_t)rr * gpr);
                if constexpr (NB == 2) {
                    u.wq[r][c][1] = dev::ldg_stream16(pk1 + rr * row_bytes);
                    u.sbw[r][c][1] = dev::ldg_stream4(sb1 + (size_t)rr * gpr);
                }
            }
        }
    };

    // Everything below reads x or writes y: wait for the preceding kernel.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (row_begin >= row_end) return;

    load_unit(ua, row_begin);
    uint32_t xr[NCH][16];
    float xs[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        load_x32(p.x, (size_t)c * kChunk + lane * 32, live[c], xr[c]);
        xs[c] = xsum32(xr[c]);
    }

    auto finish = [&](const WarpUnit<NB, R, NCH> &u, uint32_t row0) {
        float acc[R * NB];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float a = 0.0f;
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const float scale = dev::bf16_lo(u.sbw[r][c][b]), bias = dev::bf16_hi(u.sbw[r][c][b]);
                    const float dot = fmaf(-128.0f, xs[c], dot32_biased(u.wq[r][c][b], xr[c]));
                    a = fmaf(scale, dot, fmaf(bias, xs[c], a));
                }
                acc[r * NB + b] = a;
            }
        transpose_reduce<R * NB>(acc, lane);
        // After the reduction every lane holds the total of value owned_index(lane);
        // lanes 0 .. R-1 pick up row `lane` (and its gate/up partner) by shuffle.
        constexpr int V = R * NB;
        float sum[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            // value index v = r * NB + b lives in lanes whose owned_index is v: lane = bit-reverse placement
            const int want = (lane % R) * NB + b;
            int src = 0, off = 16;
#pragma unroll
            for (int sstep = V / 2; sstep >= 1; sstep >>= 1) {
                if (want & sstep) src |= off;
                off >>= 1;
            }
            sum[b] = __shfl_sync(0xffffffffu, acc[0], src);
        }
        const uint32_t row = row0 + lane;
        if (lane < R && row < sg.rows) {
            float v = sum[0];
            if (p.epi == EPI_ADD_RESID) {
                v = v + sg.resid[row];
            } else if (p.epi == EPI_GATE_UP_SILU) {
                v = dev::silu(sum[0]) * sum[NB - 1];
            } else if (p.epi == EPI_GATE_UP_GELU) {
                v = dev::gelu_pytorch_tanh(sum[0]) * sum[NB - 1];
            }
            if (p.out_bf16) {
                static_cast<uint16_t *>(sg.out)[row] = dev::f32_to_bf16_store(v);
            } else {
                static_cast<float *>(sg.out)[row] = v;
            }
        }
    };

    uint32_t row0 = row_begin;
    while (true) {
        uint32_t nxt = row0 + R;
        if (nxt < row_end) load_unit(ub, nxt);
        finish(ua, row0);
        if (nxt >= row_end) break;
        row0 = nxt;
        nxt = row0 + R;
        if (nxt < row_end) load_unit(ua, nxt);
        finish(ub, row0);
        if (nxt >= row_end) break;
        row0 = nxt;
    }
}

}  // namespace q4k
}  // namespace tessl
