// Q4 GEMV (M = 1, rows of at most 4096 columns) with the weight stream staged
// through shared memory by the bulk-copy engine.
//
// Why: a register-only streamer needs every warp to hold its next loads in
// registers, and at 168 registers per thread only ~12 warps per SM are
// resident: about 48 KiB in flight per SM, barely the bandwidth-delay product
// of HBM3e (6.5 TB/s x ~1 us / 148 SMs = 44 KiB), so the kernel measured
// latency-bound (long-scoreboard stalls, 52% issue utilisation). Here each
// warp keeps a private ring of row blocks (a few rows of packed nibbles plus
// their scale/bias pairs) in flight with `cp.async.bulk` (plain, non-multicast
// bulk copies; rows are contiguous in memory, so no tensor map is needed),
// completion counted on an mbarrier per stage. The warp reads its nibbles from
// shared memory with 128-bit loads and runs the same arithmetic as the other
// GEMV kernels (q4_gemv_kernel.cuh); its lane 0 requests the next row block
// the moment a slot has been read. A first design with one producer thread per
// block was limited by that thread (~0.3 us per stage). The whole activation
// vector stays packed in each warp's registers.
//
// Every wait on an mbarrier is bounded: after ~2 s of polling the thread sets
// the block's abort flag and the runtime's status word, every warp leaves its
// loop, gives the copies it requested a bounded chance to land, and returns.
#pragma once

#include "q4_gemv_kernel.cuh"

namespace tessl {
namespace q4k {

struct TmaSeg {
    const uint8_t *packed0;
    const uint32_t *sb0;
    const uint8_t *packed1;
    const uint32_t *sb1;
    void *out;
    const float *resid;
    uint32_t rows;
    uint32_t rb_begin;  // first row block of this bank within the launch
};

struct TmaParams {
    TmaSeg seg[3];
    int nseg;
    uint32_t total_rb;  // row blocks over all banks
    uint32_t stages;       // ring depth per warp
    uint32_t head_stages;  // stages requested before the kernel waits for its predecessor
    const uint16_t *x;
    uint32_t cols;
    uint32_t group_shift;
    int epi;
    int out_bf16;
    uint32_t *status;  // runtime status word (pinned host memory), written only on a timeout
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
/// Bounded wait: false if the phase did not complete within ~2 s or another
/// thread of the block already gave up. With `backoff_ns` the thread sleeps
/// between polls: every poll is a shared-memory request, and a few dozen warps
/// polling back to back delay the requests of the one thread whose wait is on
/// the critical path.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          uint32_t backoff_ns = 0)
{
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        if (backoff_ns) __nanosleep(backoff_ns);
        if (mbar_try(bar, parity)) return true;
        if ((i & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > 4000000000ll) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

/// NB banks (2 = gate/up), RS rows per stage and bank, NCH 1024-column chunks per row.
/// Every warp is a consumer that also feeds itself: it owns the row blocks
/// w, w + C, ... of its block's share and a private ring of `depth` stages in
/// dynamic shared memory; lane 0 requests stage j + depth as soon as the warp
/// has finished reading stage j, so no "empty" barriers are needed and the cost
/// of issuing copies is spread over all warps.
template <int NB, int RS, int NCH>
__global__ void __launch_bounds__(512, 1) q4_gemv_tma_kernel(const TmaParams p)
{
    asm volatile("griddepcontrol.launch_dependents;");
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const uint32_t cols = p.cols;
    const uint32_t gpr = cols >> p.group_shift;
    const uint32_t row_bytes = cols >> 1;
    const uint32_t sb_row_bytes = gpr * 4;
    const uint32_t stage_w_bytes = NB * RS * row_bytes;  // weights of a stage
    const uint32_t stage_bytes = stage_w_bytes + NB * RS * sb_row_bytes;
    const uint32_t D = p.stages;  // stages per warp
    const uint32_t ring = smem_u32(smem) + warp * D * stage_bytes;
    const uint32_t bars = smem_u32(smem) + nwarps * D * stage_bytes + warp * D * 8;  // full[D] of this warp
    // This block's contiguous share of the row blocks, dealt round-robin to its warps.
    const uint32_t rb_lo = (uint32_t)((uint64_t)p.total_rb * blockIdx.x / gridDim.x);
    const uint32_t rb_hi = (uint32_t)((uint64_t)p.total_rb * (blockIdx.x + 1) / gridDim.x);
    const uint32_t n_local = rb_hi - rb_lo;
    const uint32_t n_mine = n_local > (uint32_t)warp ? (n_local - warp + nwarps - 1) / nwarps : 0;

    if (threadIdx.x == 0) abort_flag = 0;
    if (lane == 0) {
        for (uint32_t s = 0; s < D; ++s) mbar_init(bars + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile int *abortp = &abort_flag;

    auto locate = [&](uint32_t rb, TmaSeg &sg, uint32_t &row0) {
        int s = 0;
        if (p.nseg > 1 && rb >= p.seg[1].rb_begin) s = 1;
        if (p.nseg > 2 && rb >= p.seg[2].rb_begin) s = 2;
        sg = p.seg[s];
        row0 = (rb - sg.rb_begin) * RS;
    };
    // Lane 0 only: request this warp's j-th row block into slot j % D.
    auto request = [&](uint32_t j) {
        TmaSeg sg;
        uint32_t row0;
        locate(rb_lo + warp + j * nwarps, sg, row0);
        const uint32_t nrows = min((uint32_t)RS, sg.rows - row0);
        const uint32_t s = j % D;
        const uint32_t dst = ring + s * stage_bytes;
        const uint32_t full = bars + 8 * s;
        mbar_expect_tx(full, NB * nrows * (row_bytes + sb_row_bytes));
        bulk_g2s(dst, sg.packed0 + (size_t)row0 * row_bytes, nrows * row_bytes, full);
        bulk_g2s(dst + stage_w_bytes, sg.sb0 + (size_t)row0 * gpr, nrows * sb_row_bytes, full);
        if constexpr (NB == 2) {
            bulk_g2s(dst + RS * row_bytes, sg.packed1 + (size_t)row0 * row_bytes, nrows * row_bytes, full);
            bulk_g2s(dst + stage_w_bytes + RS * sb_row_bytes, sg.sb1 + (size_t)row0 * gpr, nrows * sb_row_bytes,
                     full);
        }
    };

    // The weights do not depend on the preceding kernel: request the first stages now.
    uint32_t requested = 0;
    if (lane == 0) {
        const uint32_t head = min(n_mine, min(D, p.head_stages));
        for (uint32_t j = 0; j < head; ++j) request(j);
        requested = head;
    }

    bool live[NCH];
    uint32_t koff[NCH], goff[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const uint32_t k0 = c * kChunk + lane * 32;
        live[c] = k0 < cols;
        koff[c] = live[c] ? (k0 >> 1) : 0;
        goff[c] = live[c] ? (k0 >> p.group_shift) * 4 : 0;
    }
    // x is written by the preceding kernel in a decode chain: wait for it.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t xr[NCH][16];
    float xs[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) load_x32(p.x, (size_t)c * kChunk + lane * 32, live[c], xr[c]);
#pragma unroll
    for (int c = 0; c < NCH; ++c) xs[c] = xsum32(xr[c]);
    if (lane == 0) {
        const uint32_t fill = min(n_mine, D);
        for (uint32_t j = requested; j < fill; ++j) request(j);
        requested = fill;
    }

    uint32_t done = 0;  // stages whose full barrier this warp has seen complete
    for (uint32_t j = 0; j < n_mine; ++j) {
        const uint32_t s = j % D, ph = (j / D) & 1u;
        if (!mbar_wait(bars + 8 * s, ph, abortp)) {
            if (lane == 0) *(volatile uint32_t *)p.status = (2u << 24) | (j & 0xffffffu);
            break;
        }
        done = j + 1;
        const uint32_t wbase = ring + s * stage_bytes;
        const uint32_t sbase = wbase + stage_w_bytes;
        float acc[RS * NB];
#pragma unroll
        for (int r = 0; r < RS; ++r)
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float a = 0.0f;
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    // A lane past the end of the row reads real bank bytes of column 0 and drops them.
                    const uint4 w = lds128(wbase + (b * RS + r) * row_bytes + koff[c]);
                    const uint32_t pair = lds32(sbase + (b * RS + r) * sb_row_bytes + goff[c]);
                    const float scale = dev::bf16_lo(pair), bias = dev::bf16_hi(pair);
                    const float dot = fmaf(-128.0f, xs[c], dot32_biased(w, xr[c]));
                    a = live[c] ? fmaf(scale, dot, fmaf(bias, xs[c], a)) : a;
                }
                acc[r * NB + b] = a;
            }
        __syncwarp();  // every lane has finished reading the slot
        if (lane == 0 && j + D < n_mine) request(j + D);

        TmaSeg sg;
        uint32_t row0;
        locate(rb_lo + warp + j * nwarps, sg, row0);
        constexpr int V = RS * NB;
        transpose_reduce<V>(acc, lane);
        float sum[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int want = (lane % RS) * NB + b;
            int src = 0, off = 16;
#pragma unroll
            for (int st = V / 2; st >= 1; st >>= 1) {
                if (want & st) src |= off;
                off >>= 1;
            }
            sum[b] = __shfl_sync(0xffffffffu, acc[0], src);
        }
        const uint32_t row = row0 + lane;
        if (lane < RS && row < sg.rows) {
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
    }
    // Only after a timeout can copies still be in flight here: stages requested
    // but never seen complete. Give each a bounded chance to land before leaving.
    if (lane == 0 && done < n_mine) {
        const uint32_t upto = min(n_mine, done + D);
        for (uint32_t j = done; j < upto; ++j) {
            const long long t0 = clock64();
            while (!mbar_try(bars + 8 * (j % D), (j / D) & 1u)) {
                if (clock64() - t0 > 4000000000ll) break;
            }
        }
    }
}

}  // namespace q4k
}  // namespace tessl
