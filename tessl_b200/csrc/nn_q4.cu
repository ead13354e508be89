// MLX affine Q4 GEMV (M = 1) and small-batch GEMM (M <= 8) for sm_100a: the host-side wrappers that mirror
// the reference's `nn::gemv_q4_mlx_*`, `nn::gemm_q4_mlx` and `nn::embed_lookup_q4_mlx` (src/nn.rs:3592-4619 of
// the reference project): validation in the reference's order and wording, the choice of kernel and
// instantiation, the launch.
//
// Kernels: q4_gemv_mma.cuh (the default: dot products on the tensor cores, bulk-copy ring; also the MLX Q8 mode
// and the column-sharded launches that exchange their outputs over NVLink), and the FMA-pipe fallbacks
// q4_gemv_tma.cuh, q4_gemv_warp.cuh, q4_gemv_main.cuh / q4_gemv_kernel.cuh for the shapes it does not take.
#include "q4_gemv_main.cuh"
#include "q4_gemv_warp.cuh"
#include "q4_gemv_tma.cuh"
#include "q4_gemv_mma.cuh"

#include <cstdio>
#include <cstdlib>
#include "runtime.h"

namespace tessl {
namespace {

using q4k::EPI_ADD_RESID;
using q4k::EPI_GATE_UP_GELU;
using q4k::EPI_GATE_UP_SILU;
using q4k::EPI_STORE;
using Q4Seg = q4k::Seg;
using Q4GemvParams = q4k::Params;

__global__ void swiglu_kernel(const float *gate, const float *up, void *out, uint32_t n, int out_bf16, int gelu)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = (gelu ? dev::gelu_pytorch_tanh(gate[i]) : dev::silu(gate[i])) * up[i];
    if (out_bf16) {
        static_cast<uint16_t *>(out)[i] = dev::f32_to_bf16_store(v);
    } else {
        static_cast<float *>(out)[i] = v;
    }
}

__global__ void q4_unpack_kernel(const uint8_t *packed, uint8_t *out, uint64_t n_bytes)
{
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_bytes) return;
    const uint8_t b = packed[i];
    out[2 * i] = b & 0x0f;
    out[2 * i + 1] = b >> 4;
}

/// Geometry of the staged layout for rows of `cols` columns and groups of `group` (see q4_gemv_mma.cuh).
struct StagedGeom {
    uint32_t row_bytes, pair_pitch, sb_row_bytes, unit_bytes;
};
__host__ __device__ inline StagedGeom staged_geom(uint32_t cols, uint32_t group)
{
    StagedGeom g;
    g.row_bytes = cols / 2;
    g.pair_pitch = 2 * g.row_bytes + q4m::kRowPad;
    g.sb_row_bytes = (cols / group) * 4;
    g.unit_bytes = 4 * g.pair_pitch + 8 * g.sb_row_bytes;
    return g;
}

/// One thread per 16 bytes of the staged image: a piece of a packed row, of a pad, or of a scale/bias row.
__global__ void q4_repack_staged_kernel(const uint4 *packed, const uint4 *sb, uint4 *out, uint32_t rows, uint32_t cols,
                                        uint32_t group, uint64_t n16)
{
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n16) return;
    const StagedGeom g = staged_geom(cols, group);
    const uint64_t byte = i * 16;
    const uint32_t unit = (uint32_t)(byte / g.unit_bytes), o = (uint32_t)(byte % g.unit_bytes);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (o < 4 * g.pair_pitch) {
        const uint32_t pair = o / g.pair_pitch, within = o % g.pair_pitch;
        if (within < 2 * g.row_bytes) {
            const uint32_t row = 8 * unit + 2 * pair + within / g.row_bytes;
            if (row < rows) v = packed[((size_t)row * g.row_bytes + within % g.row_bytes) / 16];
        }
    } else {
        const uint32_t so = o - 4 * g.pair_pitch;
        const uint32_t row = 8 * unit + so / g.sb_row_bytes;
        if (row < rows) v = sb[((size_t)row * g.sb_row_bytes + so % g.sb_row_bytes) / 16];
    }
    out[i] = v;
}

__global__ void q4_dequant_kernel(const uint8_t *packed, const uint32_t *sb, float *out, uint32_t rows, uint32_t cols,
                                  uint32_t group_shift)
{
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;  // byte index
    if (i >= (uint64_t)rows * cols / 2) return;
    const uint64_t e = 2 * i;
    const uint32_t row = (uint32_t)(e / cols), col = (uint32_t)(e % cols);
    const uint32_t pair = sb[(size_t)row * (cols >> group_shift) + (col >> group_shift)];
    const float scale = dev::bf16_lo(pair), bias = dev::bf16_hi(pair);
    const uint8_t b = packed[i];
    // Separate multiply and add, as the reference's host dequant (scale * q is exact anyway).
    out[e] = __fadd_rn(__fmul_rn(scale, (float)(b & 0x0f)), bias);
    out[e + 1] = __fadd_rn(__fmul_rn(scale, (float)(b >> 4)), bias);
}

/// One thread per 32 consecutive columns of one token's row (16 packed bytes, never more than one
/// quantization group): a 128-bit load of the nibbles, one scale/bias pair, eight 128-bit stores.
/// A token id outside the table gives a row of zeros (kernels/embed_lookup.metal:24-27 of the
/// reference project).
__global__ void embed_lookup_q4_mlx_kernel(const uint8_t *packed, const uint32_t *sb, const uint32_t *token_ids, float *out,
                                           uint32_t hidden, uint32_t group_shift, uint32_t vocab, uint64_t total32)
{
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total32) return;
    const uint32_t per_row = hidden / 32;
    const uint32_t m = (uint32_t)(i / per_row), c = (uint32_t)(i % per_row);
    const uint32_t tid = token_ids[m];
    float4 *o = reinterpret_cast<float4 *>(out + (size_t)m * hidden + (size_t)c * 32);
    if (tid >= vocab) {
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        return;
    }
    const uint4 w = dev::ldg_stream16(packed + (size_t)tid * (hidden / 2) + (size_t)c * 16);
    const uint32_t pair = sb[(size_t)tid * (hidden >> group_shift) + ((c * 32) >> group_shift)];
    const float scale = dev::bf16_lo(pair), bias = dev::bf16_hi(pair);
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float v[8];
#pragma unroll
        for (int n = 0; n < 8; ++n) v[n] = __fadd_rn(__fmul_rn(scale, (float)((words[k] >> (4 * n)) & 15u)), bias);
        o[2 * k] = make_float4(v[0], v[1], v[2], v[3]);
        o[2 * k + 1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

uint32_t log2_u32(uint32_t v)
{
    uint32_t s = 0;
    while ((1u << s) < v) ++s;
    return s;
}

template <int M, int NB, int R, int NCH>
Result launch_one(TesslRuntime *rt, Q4GemvParams &p, int warps)
{
    auto kernel = q4k::q4_gemv_kernel<M, NB, R, NCH>;
    uint32_t groups = 0;
    for (int s = 0; s < p.nseg; ++s) {
        p.seg[s].group_begin = groups;
        groups += (p.seg[s].rows + R - 1) / R;
    }
    p.ngroups = groups;
    if (groups == 0) return ok();
    // Persistent grid: as many blocks as stay resident, each walking its share of the groups.
    static int per_sm[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (per_sm[warps] == 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, warps * 32, 0);
        if (e != cudaSuccess || n < 1) n = 1;
        per_sm[warps] = n;
    }
    const uint32_t grid = std::min<uint32_t>(groups, (uint32_t)(rt->sm_count * per_sm[warps]));
    kernel<<<grid, warps * 32, 0, rt->stream>>>(p);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "q4_gemv launch");
}

template <int NB, int R, int NCH>
Result launch_warp(TesslRuntime *rt, const Q4GemvParams &p)
{
    auto kernel = q4k::q4_gemv_warp_kernel<NB, R, NCH>;
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 32, 0);
        per_sm = (e != cudaSuccess || n < 1) ? 1 : n;
    }
    q4k::WarpParams wp{};
    uint64_t total_rows = 0;
    for (int s = 0; s < p.nseg; ++s) total_rows += p.seg[s].rows;
    if (total_rows == 0) return ok();
    // One wave: every warp gets the same number of consecutive rows.
    const uint64_t capacity = (uint64_t)rt->sm_count * per_sm;
    uint64_t r = (total_rows + capacity - 1) / capacity;
    r = (r + R - 1) / R * R;
    uint32_t blocks = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const Q4Seg &a = p.seg[s];
        wp.seg[s] = q4k::WarpSeg{a.packed0, a.sb0, a.packed1, a.sb1, a.out, a.resid, a.rows, blocks};
        blocks += (uint32_t)((a.rows + r - 1) / r);
    }
    wp.nseg = p.nseg;
    wp.rows_per_block = (uint32_t)r;
    wp.x = p.x, wp.cols = p.cols, wp.group_shift = p.group_shift, wp.epi = p.epi, wp.out_bf16 = p.out_bf16;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks), cfg.blockDim = dim3(32), cfg.dynamicSmemBytes = 0, cfg.stream = rt->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, wp);
    rt->dispatch_count += 1;
    return cuda_check(rt, e, "q4_gemv launch");
}

/// Experiment knobs for the staged kernel: "consumers,ring_kib,blocks_per_sm".
struct TmaCfg {
    int consumers = 16, ring_kib = 148, blocks_per_sm = 1, head_stages = 1, enabled = 1;
};
const TmaCfg &tma_cfg()
{
    static TmaCfg c = [] {
        TmaCfg t;
        if (const char *e = std::getenv("TESSL_B200_GEMV_TMA")) {
            int a = 0, b = 0, d = 0, h = 0;
            const int n = std::sscanf(e, "%d,%d,%d,%d", &a, &b, &d, &h);
            if (n >= 4 && h > 0) t.head_stages = h;
            if (n >= 1 && a == 0) t.enabled = 0;
            if (n >= 1 && a > 0) t.consumers = std::min(a, 16);
            if (n >= 2 && b > 0) t.ring_kib = b;
            if (n >= 3 && d > 0) t.blocks_per_sm = d;
        }
        return t;
    }();
    return c;
}

template <int NB, int RS, int NCH>
Result launch_tma(TesslRuntime *rt, const Q4GemvParams &p)
{
    auto kernel = q4k::q4_gemv_tma_kernel<NB, RS, NCH>;
    const TmaCfg &cfg = tma_cfg();
    q4k::TmaParams tp{};
    uint32_t rb = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const Q4Seg &a = p.seg[s];
        tp.seg[s] = q4k::TmaSeg{a.packed0, a.sb0, a.packed1, a.sb1, a.out, a.resid, a.rows, rb};
        rb += (a.rows + RS - 1) / RS;
    }
    if (rb == 0) return ok();
    tp.nseg = p.nseg, tp.total_rb = rb;
    tp.x = p.x, tp.cols = p.cols, tp.group_shift = p.group_shift, tp.epi = p.epi, tp.out_bf16 = p.out_bf16;
    tp.status = rt->status_dev;
    const uint32_t stage_bytes = NB * RS * ((p.cols >> 1) + (p.cols >> p.group_shift) * 4);
    const uint32_t warps = (uint32_t)cfg.consumers;
    const uint32_t stages = std::max<uint32_t>(1u, (uint32_t)cfg.ring_kib * 1024u / (stage_bytes * warps));
    tp.stages = stages;
    tp.head_stages = (uint32_t)cfg.head_stages;
    const size_t smem = (size_t)warps * stages * (stage_bytes + 8);
    TESSL_TRY(smem_opt_in(rt, reinterpret_cast<const void *>(kernel), smem, "q4_gemv_tma: shared memory opt-in"));
    const uint32_t grid = std::min<uint32_t>(rb, (uint32_t)(rt->sm_count * cfg.blocks_per_sm));
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(grid), lc.blockDim = dim3(cfg.consumers * 32), lc.dynamicSmemBytes = smem;
    lc.stream = rt->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr, lc.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, kernel, tp);
    rt->dispatch_count += 1;
    return cuda_check(rt, e, "q4_gemv launch");
}

/// The tensor-core kernel (q4_gemv_mma.cuh): rows of 1024, 2048 or 4096 columns
/// whose sixteenth holds whole quantization groups, scale/bias rows that a bulk
/// copy can fetch. TESSL_B200_GEMV_MMA=0 turns it off (tuning runs).
bool mma_enabled()
{
    static int on = -1;
    if (on < 0) {
        const char *e = std::getenv("TESSL_B200_GEMV_MMA");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

bool mma_ok(const Q4GemvParams &p)
{
    if (!mma_enabled()) return false;
    if (p.cols != 1024 && p.cols != 2048 && p.cols != 4096) return false;
    if (p.group_shift < 5 || p.group_shift > 7) return false;
    if (((p.cols / 16) >> p.group_shift) == 0) return false;
    for (int s = 0; s < p.nseg && !p.staged; ++s) {
        const Q4Seg &a = p.seg[s];
        if (((uintptr_t)a.sb0 & 15u) || (a.sb1 && ((uintptr_t)a.sb1 & 15u))) return false;
    }
    return true;
}

/// A launch over a window of `cols` columns of longer rows (one K chunk): distances in global
/// memory between packed rows and scale/bias rows (bytes) and between batch rows of x (elements).
/// Zeros: dense rows.
struct MmaWindow {
    uint32_t row_pitch = 0, sb_pitch = 0, x_pitch = 0;
};

/// Shared memory one block of the tensor-core GEMV may use: the per-block maximum of sm_100 less the kernel's few
/// static bytes.
constexpr uint32_t kMmaSmemBudget = 232448u - 512u;

template <int SW, int WPG, int NB, bool BATCH, bool Q8 = false, int NWIN = 1, int ROWS = 16, bool STAGED = false>
Result launch_mma_one(TesslRuntime *rt, const Q4GemvParams &p, int m, const MmaWindow &w = MmaWindow{})
{
    auto kernel = q4m::q4_gemv_mma_kernel<SW, WPG, NB, BATCH, Q8, NWIN, ROWS, STAGED>;
    constexpr uint32_t RPB = ROWS / NB;
    q4m::Params mp{};
    uint32_t rb = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const Q4Seg &a = p.seg[s];
        mp.seg[s] = q4m::Seg{a.packed0, a.sb0, a.packed1, a.sb1, a.out, a.resid, a.rows, rb};
        rb += (a.rows + RPB - 1) / RPB;
    }
    if (rb == 0) return ok();
    mp.nseg = p.nseg, mp.total_rb = rb;
    mp.x = p.x, mp.m = (uint32_t)m, mp.cols = p.cols, mp.group_shift = p.group_shift;
    mp.epi = p.epi, mp.out_bf16 = p.out_bf16;
    mp.row_pitch = w.row_pitch ? w.row_pitch : p.cols >> 1;
    mp.sb_pitch = w.sb_pitch ? w.sb_pitch : (p.cols >> p.group_shift) * 4;
    mp.x_pitch = w.x_pitch ? w.x_pitch : (Q8 ? p.cols >> 1 : p.cols);
    mp.status = rt->status_dev;
    if ((p.staged != 0) != STAGED) return "q4_gemv: the staged layout runs on the one-row Q4 kernel only";
    if (p.peer) {
        const TesslPeerGather &g = *static_cast<const TesslPeerGather *>(p.peer);
        if (BATCH || Q8 || p.nseg != 1) return "q4_gemv: a sharded launch has one bank (or one gate/up pair) and one row of x";
        for (uint32_t r = 0; r < g.world; ++r) {
            mp.peer.out[r] = static_cast<uint8_t *>(g.buffers[r]) + (size_t)g.rank * g.bytes_per_rank;
            mp.peer.flags[r] = g.flags[r];
        }
        mp.peer.rank = g.rank, mp.peer.world = g.world, mp.peer_world = g.world;
        mp.peer.wait_clocks = rt->peer_wait_clocks ? (long long)rt->peer_wait_clocks : kPeerWaitClocks;
        mp.peer.defer = p.peer_defer ? 1u : 0u;
    }
    if (p.xwait) {
        const TesslPeerGather &g = *static_cast<const TesslPeerGather *>(p.xwait);
        if (BATCH || Q8) return "q4_gemv: a gathered x is one row";
        mp.xwait.flags = g.flags[g.rank];
        mp.xwait.rank = g.rank, mp.xwait.world = g.world, mp.xwait_world = g.world;
        mp.xwait.wait_clocks = rt->peer_wait_clocks ? (long long)rt->peer_wait_clocks : kPeerWaitClocks;
    }
    const uint32_t gpr = p.cols >> p.group_shift;
    const uint32_t part = BATCH ? q4m::kConsumers * 16 * 8 * 4 : q4m::kConsumers * 16 * 4;
    const uint32_t stage_bytes = ROWS * ((p.cols >> 1) + q4m::kRowPad) + ROWS * gpr * 4 + part;
    // the warps' staged slices of x: only the Q4 kernel for one row of x stages them
    const uint32_t x_stage = 32 + ((BATCH || Q8) ? 0u : q4m::kConsumers * q4m::kXStageBytes * NWIN);
    uint32_t stages = std::min<uint32_t>(8u, (kMmaSmemBudget - x_stage) / (stage_bytes + 24));
    if (stages < 2) return "q4_gemv_mma: the ring does not fit two stages";
    mp.stages = stages;
    const size_t smem = (size_t)stages * (stage_bytes + 24) + x_stage;
    TESSL_TRY(smem_opt_in(rt, reinterpret_cast<const void *>(kernel), smem, "q4_gemv_mma: shared memory opt-in", true));
    const uint32_t grid = std::min<uint32_t>(rb, (uint32_t)rt->sm_count);
    {
        const uint64_t step = (((uint64_t)rb << 32) + grid - 1) / grid;  // rb <= 2^32 - 1 and grid <= rb: step fits 64 bits
        mp.rb_step_lo = (uint32_t)step, mp.rb_step_hi = (uint32_t)(step >> 32);
    }
    // four rows per bulk copy wherever two row pairs are adjacent in memory (one bank, dense rows): 151936 x 4096
    // 58.8 -> 52.7 us, 6144 x 4096 5.30 -> 5.05 us, 12288 x 4096 8.00 -> 7.90 us on one box, back to back.
    // Not for Q8: its row pair is already 8 KB, and 16 KB copies ran 14336 x 4096 in 17.0 us against 14.5.
    mp.quads = (!BATCH && !Q8 && NWIN == 1 && w.row_pitch == 0 && !p.staged) ? 1u : 0u;
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(grid), lc.blockDim = dim3(q4m::kThreads), lc.dynamicSmemBytes = smem;
    lc.stream = rt->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr, lc.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, kernel, mp);
    rt->dispatch_count += 1;
    return cuda_check(rt, e, "q4_gemv launch");
}

template <int SW, int WPG>
Result launch_mma_sw(TesslRuntime *rt, const Q4GemvParams &p, int m, int nb, const MmaWindow &w)
{
    if (p.staged) {
        if (m != 1 || w.row_pitch != 0) return "q4_gemv: the staged layout runs on the one-row Q4 kernel only";
        if (nb == 2) return launch_mma_one<SW, WPG, 2, false, false, 1, 16, true>(rt, p, m, w);
        return launch_mma_one<SW, WPG, 1, false, false, 1, 16, true>(rt, p, m, w);
    }
    if (nb == 2) return launch_mma_one<SW, WPG, 2, false>(rt, p, m, w);
    if (m == 1) return launch_mma_one<SW, WPG, 1, false>(rt, p, m, w);
    return launch_mma_one<SW, WPG, 1, true>(rt, p, m, w);
}

Result launch_mma(TesslRuntime *rt, const Q4GemvParams &p, int m, int nb, const MmaWindow &w = MmaWindow{})
{
    const int sw = (int)(p.cols / 512), wpg = 1 << (p.group_shift - 5);
    if (sw == 8) {
        if (wpg == 1) return launch_mma_sw<8, 1>(rt, p, m, nb, w);
        if (wpg == 2) return launch_mma_sw<8, 2>(rt, p, m, nb, w);
        return launch_mma_sw<8, 4>(rt, p, m, nb, w);
    }
    if (sw == 4) {
        if (wpg == 1) return launch_mma_sw<4, 1>(rt, p, m, nb, w);
        if (wpg == 2) return launch_mma_sw<4, 2>(rt, p, m, nb, w);
        return launch_mma_sw<4, 4>(rt, p, m, nb, w);
    }
    if (wpg == 1) return launch_mma_sw<2, 1>(rt, p, m, nb, w);
    return launch_mma_sw<2, 2>(rt, p, m, nb, w);
}

/// One row of x over rows of 8192 or 12288 columns (a 4096 x 12288 down projection): the tensor-core kernel
/// with every stage holding whole long rows, the warps walking the 4096-column windows inside it. Two
/// stages fit in shared memory (of 16 rows at 8192 columns, of 14 at 12288). Taken for every M = 1 form at
/// these widths, whatever the row count, so that a row's summation order still depends on K and G alone.
bool mma_long_ok(const Q4GemvParams &p, int m)
{
    if (!mma_enabled() || m != 1) return false;
    if (p.cols != 8192 && p.cols != 12288) return false;
    if (p.group_shift < 5 || p.group_shift > 7) return false;
    for (int s = 0; s < p.nseg; ++s) {
        const Q4Seg &a = p.seg[s];
        if (((uintptr_t)a.sb0 & 15u) || (a.sb1 && ((uintptr_t)a.sb1 & 15u))) return false;
    }
    return true;
}

Result launch_mma_long(TesslRuntime *rt, const Q4GemvParams &p)
{
    const int wpg = 1 << (p.group_shift - 5);
    if (p.cols == 8192) {
        if (wpg == 1) return launch_mma_one<8, 1, 1, false, false, 2, 16>(rt, p, 1);
        if (wpg == 2) return launch_mma_one<8, 2, 1, false, false, 2, 16>(rt, p, 1);
        return launch_mma_one<8, 4, 1, false, false, 2, 16>(rt, p, 1);
    }
    if (wpg == 1) return launch_mma_one<8, 1, 1, false, false, 3, 14>(rt, p, 1);
    if (wpg == 2) return launch_mma_one<8, 2, 1, false, false, 3, 14>(rt, p, 1);
    return launch_mma_one<8, 4, 1, false, false, 3, 14>(rt, p, 1);
}

/// Batches of 3..8 rows over rows longer than the tensor-core kernel's 4096 columns (a 12288-column
/// down projection in batched decode): one launch of that kernel per window of 4096 columns, each
/// after the first adding to the f32 result of those before it (the kernel's add-residual epilogue
/// with the output as the residual; launches on one stream are ordered). The FMA-pipe kernel this
/// replaces costs one pass per batch row (4096 x 12288: 65 us at M = 8 against 21 us here; at
/// M = 2 it is still the faster one, 17 us against 20 us). Returns false if the call does not fit.
bool launch_mma_windows(TesslRuntime *rt, const Q4GemvParams &p, int m, int nb, Result &res)
{
    constexpr uint32_t W = 4096;
    if (m < 3 || m > 8 || nb != 1 || p.nseg != 1 || p.cols <= W || p.cols % W != 0 || p.out_bf16) return false;
    if (p.epi != q4k::EPI_STORE) return false;  // a residual is added once, after the whole sum: not expressible here
    Q4GemvParams q = p;
    q.cols = W;
    if (!mma_ok(q)) return false;
    MmaWindow w;
    w.row_pitch = p.cols >> 1, w.sb_pitch = (p.cols >> p.group_shift) * 4, w.x_pitch = p.cols;
    for (uint32_t c = 0; c < p.cols / W; ++c) {
        q.x = p.x + (size_t)c * W;
        q.seg[0].packed0 = p.seg[0].packed0 + (size_t)c * (W / 2);
        q.seg[0].sb0 = p.seg[0].sb0 + (size_t)c * (W >> p.group_shift);
        if (c > 0) q.epi = q4k::EPI_ADD_RESID, q.seg[0].resid = static_cast<const float *>(p.seg[0].out);
        res = launch_mma(rt, q, m, 1, w);
        if (!res.empty()) return true;
    }
    return true;
}

template <int SW, int WPG>
Result launch_mma_q8_sw(TesslRuntime *rt, const Q4GemvParams &p, int m)
{
    // 4096 codes per row: a 16-row stage with the batch's partial sums is 77 KB and only two fit; 10-row stages
    // (part of each MMA idle, which this format can afford: one MMA per 8 bytes of weights) give four. A stage's
    // compute does not depend on its height, so fewer and taller stages win as long as the ring stays deep enough:
    // 14336 x 4096 at M = 2 / 4 / 8: 8 rows (five stages) 16.5 / 17.0 / 17.5 us, 10 rows 14.6 / 15.0 / 15.6 us,
    // 12 rows (three stages) 16.8 / 17.1 / 17.7 us.
    if (SW == 16 && m > 1) return launch_mma_one<SW, WPG, 1, true, true, 1, 10>(rt, p, m);
    if (SW == 16 && m == 1) {
        // One row of x over 4096 codes per row is bound by the stream, not by the consumers (a stage's compute does
        // not depend on its height, its bytes do), so the stage height that leaves the shortest tail wins: the
        // busiest SM streams ceil(stages / SMs) x height rows. 14336 rows: 16 -> 14.4 us, 12 -> 14.05, 10 -> 13.7,
        // 8 -> 15.4 (half of every MMA idle begins to cost). Ties go to the taller stage.
        uint32_t rows = 0;
        for (int s = 0; s < p.nseg; ++s) rows += p.seg[s].rows;
        const uint32_t sms = (uint32_t)rt->sm_count;
        auto tail = [&](uint32_t h) { return (((rows + h - 1) / h + sms - 1) / sms) * h; };
        if (tail(10) < tail(16) && tail(10) < tail(12)) return launch_mma_one<SW, WPG, 1, false, true, 1, 10>(rt, p, m);
        if (tail(12) < tail(16)) return launch_mma_one<SW, WPG, 1, false, true, 1, 12>(rt, p, m);
    }
    if (m == 1) return launch_mma_one<SW, WPG, 1, false, true>(rt, p, m);
    return launch_mma_one<SW, WPG, 1, true, true>(rt, p, m);
}

/// The staged kernel needs every bulk copy 16-byte aligned and sized.
bool tma_ok(const Q4GemvParams &p)
{
    if (!tma_cfg().enabled) return false;
    if (p.cols == 0 || p.cols > 4096) return false;
    if ((((p.cols >> p.group_shift) * 4) & 15u) != 0) return false;
    for (int s = 0; s < p.nseg; ++s) {
        const Q4Seg &a = p.seg[s];
        if (((uintptr_t)a.sb0 & 15u) || (a.sb1 && ((uintptr_t)a.sb1 & 15u))) return false;
    }
    return true;
}

/// Picks the split of K over warps (a function of `cols` only, so a row's
/// summation order never depends on the launch) and the matching instantiation.
Result launch_q4_gemv(TesslRuntime *rt, Q4GemvParams p, int m, int nb)
{
    if (p.xwait && !(m == 1 && (mma_ok(p) || mma_long_ok(p, m)))) {
        // a width the tensor-core kernel does not take: the wait as a launch of its own, then whichever kernel serves it
        const TesslPeerGather *g = static_cast<const TesslPeerGather *>(p.xwait);
        p.xwait = nullptr;
        TESSL_TRY(nn::peer_wait(rt, *g));
        return launch_q4_gemv(rt, p, m, nb);
    }
    if (p.peer && !(m == 1 && (mma_ok(p) || (mma_long_ok(p, m) && nb == 1)))) {
        // shapes the tensor-core kernel does not take: the slice by whichever kernel serves it, then the
        // stand-alone exchange (same flag words, same result)
        const TesslPeerGather *g = static_cast<const TesslPeerGather *>(p.peer);
        p.peer = nullptr;
        TESSL_TRY(launch_q4_gemv(rt, p, m, nb));
        return nn::peer_gather(rt, *g);
    }
    const uint32_t nchunks = std::max<uint32_t>(1u, (p.cols + q4k::kChunk - 1) / q4k::kChunk);
    if (p.staged && !(m == 1 && mma_ok(p)))
        return "q4_gemv: the staged layout needs the tensor-core GEMV kernel (one row of x, rows of 1024, 2048 or 4096 columns)";
    if (m >= 1 && m <= 8 && (nb == 1 || m == 1) && mma_ok(p)) return launch_mma(rt, p, m, nb);
    if (mma_long_ok(p, m)) {
        // The kernel takes one bank per launch at these widths. The bank-routed forms run as one launch per
        // bank, the gate/up forms as two launches into scratch and the activation kernel: what the fused
        // launches are defined to equal bit for bit.
        if (nb == 1) {
            for (int sidx = 0; sidx < p.nseg; ++sidx) {
                Q4GemvParams q = p;
                q.seg[0] = p.seg[sidx], q.nseg = 1;
                TESSL_TRY(launch_mma_long(rt, q));
            }
            return ok();
        }
        const uint32_t rows = p.seg[0].rows;
        void *tmp = nullptr;
        TESSL_TRY(scratch_reserve(rt, (size_t)rows * 8, &tmp));
        float *g = static_cast<float *>(tmp), *u = g + rows;
        Q4GemvParams q = p;
        q.epi = EPI_STORE, q.out_bf16 = 0, q.peer = nullptr;
        q.seg[0].packed1 = nullptr, q.seg[0].sb1 = nullptr, q.seg[0].out = g;
        TESSL_TRY(launch_mma_long(rt, q));
        q.seg[0].packed0 = p.seg[0].packed1, q.seg[0].sb0 = p.seg[0].sb1, q.seg[0].out = u;
        TESSL_TRY(launch_mma_long(rt, q));
        swiglu_kernel<<<(rows + 255) / 256, 256, 0, rt->stream>>>(g, u, p.seg[0].out, rows, p.out_bf16,
                                                                  p.epi == EPI_GATE_UP_GELU ? 1 : 0);
        rt->dispatch_count += 1;
        TESSL_TRY(cuda_check(rt, cudaGetLastError(), "gate/up activation launch"));
        if (p.peer) return nn::peer_gather(rt, *static_cast<const TesslPeerGather *>(p.peer));
        return ok();
    }
    {
        Result res = ok();
        if (launch_mma_windows(rt, p, m, nb, res)) return res;
    }
    if (m == 1 && nchunks <= 4 && tma_ok(p)) {
        if (nb == 1) {
            if (nchunks == 1) return launch_tma<1, 8, 1>(rt, p);
            if (nchunks == 2) return launch_tma<1, 4, 2>(rt, p);
            if (nchunks == 3) return launch_tma<1, 2, 3>(rt, p);
            return launch_tma<1, 2, 4>(rt, p);
        }
        if (nchunks == 1) return launch_tma<2, 4, 1>(rt, p);
        if (nchunks == 2) return launch_tma<2, 2, 2>(rt, p);
        if (nchunks == 3) return launch_tma<2, 1, 3>(rt, p);
        return launch_tma<2, 1, 4>(rt, p);
    }
    if (m == 1 && nchunks <= 4) {
        // Rows of at most 4096 columns: one warp keeps all of x resident.
        if (nb == 1) {
            if (nchunks == 1) return launch_warp<1, 8, 1>(rt, p);
            if (nchunks == 2) return launch_warp<1, 4, 2>(rt, p);
            if (nchunks == 3) return launch_warp<1, 2, 3>(rt, p);
            return launch_warp<1, 2, 4>(rt, p);
        }
        if (nchunks == 1) return launch_warp<2, 4, 1>(rt, p);
        if (nchunks == 2) return launch_warp<2, 2, 2>(rt, p);
        if (nchunks == 3) return launch_warp<2, 1, 3>(rt, p);
        return launch_warp<2, 1, 4>(rt, p);
    }
    if (m == 1) {
        int warps, nch;
        if (nchunks <= 4) {
            warps = (int)nchunks, nch = 1;
        } else if (nchunks <= 16) {
            warps = (int)(nchunks + 1) / 2, nch = 2;
        } else if (nchunks <= 32) {
            warps = (int)(nchunks + 3) / 4, nch = 4;
        } else {
            warps = 8, nch = 0;
        }
        if (nb == 1) {
            if (nch == 1) return launch_one<1, 1, 8, 1>(rt, p, warps);
            if (nch == 2) return launch_one<1, 1, 4, 2>(rt, p, warps);
            if (nch == 4) return launch_one<1, 1, 2, 4>(rt, p, warps);
            return launch_one<1, 1, 8, 0>(rt, p, warps);
        }
        if (nch == 1) return launch_one<1, 2, 4, 1>(rt, p, warps);
        if (nch == 2) return launch_one<1, 2, 2, 2>(rt, p, warps);
        if (nch == 4) return launch_one<1, 2, 1, 4>(rt, p, warps);
        return launch_one<1, 2, 4, 0>(rt, p, warps);
    }
    const int warps = (int)std::min<uint32_t>(4u, nchunks);
    switch (m) {
    case 2: return launch_one<2, 1, 4, 0>(rt, p, warps);
    case 3: return launch_one<3, 1, 2, 0>(rt, p, warps);
    case 4: return launch_one<4, 1, 2, 0>(rt, p, warps);
    case 5: return launch_one<5, 1, 2, 0>(rt, p, warps);
    case 6: return launch_one<6, 1, 2, 0>(rt, p, warps);
    case 7: return launch_one<7, 1, 2, 0>(rt, p, warps);
    case 8: return launch_one<8, 1, 2, 0>(rt, p, warps);
    default: return fmt("q4_gemv: no kernel for m=%d", m);
    }
}

Q4Seg make_seg(const TesslQ4MlxBank &b0, const TesslQ4MlxBank *b1, const TesslBuf &out, const TesslBuf *resid,
               uint32_t rows)
{
    Q4Seg s{};
    s.packed0 = static_cast<const uint8_t *>(b0.packed.ptr);
    s.sb0 = static_cast<const uint32_t *>(b0.scales_biases.ptr);
    s.packed1 = b1 ? static_cast<const uint8_t *>(b1->packed.ptr) : nullptr;
    s.sb1 = b1 ? static_cast<const uint32_t *>(b1->scales_biases.ptr) : nullptr;
    s.out = out.ptr;
    s.resid = resid ? static_cast<const float *>(resid->ptr) : nullptr;
    s.rows = rows;
    return s;
}

bool staged_domain(uint32_t cols, uint32_t group)
{
    if (cols != 1024 && cols != 2048 && cols != 4096) return false;
    if (group != 32 && group != 64 && group != 128) return false;
    return (cols / 16) / group >= 1;
}

Result check_alignment(const TesslQ4MlxBank &b, const std::string &what);

/// The bank checks of an entry that takes either layout: the reference's for a row-major bank, size,
/// domain and alignment of the image for a staged one.
Result bank_validate_layout(const TesslQ4MlxBank &bank, const TesslQuantShape &shape, uint32_t layout, const std::string &what)
{
    if (layout != TESSL_Q4_B200_STAGED) return q4_bank_validate(bank, shape, what);
    TESSL_TRY(quant_shape_validate(shape, what));
    if (!staged_domain(shape.cols, shape.group_size))
        return fmt("%s: the B200 staged layout exists for rows of 1024, 2048 or 4096 columns and groups of 32, 64 or 128 "
                   "(got %u columns, group %u)", what.c_str(), shape.cols, shape.group_size);
    TESSL_TRY(require(bank.packed, nn::q4_mlx_staged_bytes(shape.rows, shape.cols, shape.group_size), 1, what + " staged image"));
    return require_aligned16(bank.packed, what + " staged image");
}

Result check_alignment(const TesslQ4MlxBank &b, const std::string &what)
{
    TESSL_TRY(require_aligned16(b.packed, what + " packed"));
    if (((uintptr_t)b.scales_biases.ptr & 3u) != 0)
        return fmt("%s scales_biases: device pointer must be 4-byte aligned", what.c_str());
    return ok();
}

}  // namespace

namespace nn {

/// MLX Q8 (unsigned codes, bf16 pairs, bf16 x, M <= 8) on the tensor-core GEMV kernel: a row of `cols`
/// codes is laid out and staged like a row of 2 cols nibbles with groups of 2 group_size (the kernel's sizes
/// are in nibbles); the codes themselves go to the MMA as bf16 bit patterns, two per register. `*handled` is false when the shape is
/// not one the kernel is built for (the caller then uses its FMA-pipe kernel).
Result q8_mlx_mma(TesslRuntime *rt, const TesslBuf &codes, const TesslBuf &sb, const TesslBuf &x_bf16, const TesslBuf &y,
                  uint32_t rows, uint32_t cols, uint32_t group_size, uint32_t m, OutKind out, bool *handled)
{
    *handled = false;
    if (!mma_enabled()) return ok();
    if (m < 1) return ok();
    if (cols != 512 && cols != 1024 && cols != 2048 && cols != 4096) return ok();
    if (group_size != 32 && group_size != 64) return ok();
    if (((uintptr_t)sb.ptr & 15u) != 0 || ((uintptr_t)x_bf16.ptr & 7u) != 0) return ok();
    if (((2 * cols / 16) / (2 * group_size)) == 0) return ok();  // a warp's slice holds whole groups
    *handled = true;
    Q4GemvParams p{};
    p.nseg = 1;
    p.seg[0] = Q4Seg{};
    p.seg[0].packed0 = static_cast<const uint8_t *>(codes.ptr);
    p.seg[0].sb0 = static_cast<const uint32_t *>(sb.ptr);
    p.seg[0].out = y.ptr;
    p.seg[0].rows = rows;
    p.x = static_cast<const uint16_t *>(x_bf16.ptr);
    p.cols = 2 * cols;
    p.group_shift = log2_u32(2 * group_size);
    p.epi = EPI_STORE;
    p.out_bf16 = out == OUT_BF16;
    const int sw = (int)(p.cols / 512);
    const bool g64 = group_size == 64;  // 128 nibbles: 4 words per lane and group; 32 codes: 2
    switch (sw) {
    case 2: return g64 ? launch_mma_q8_sw<2, 2>(rt, p, (int)m) : launch_mma_q8_sw<2, 2>(rt, p, (int)m);
    case 4: return g64 ? launch_mma_q8_sw<4, 4>(rt, p, (int)m) : launch_mma_q8_sw<4, 2>(rt, p, (int)m);
    case 8: return g64 ? launch_mma_q8_sw<8, 4>(rt, p, (int)m) : launch_mma_q8_sw<8, 2>(rt, p, (int)m);
    default: return g64 ? launch_mma_q8_sw<16, 4>(rt, p, (int)m) : launch_mma_q8_sw<16, 2>(rt, p, (int)m);
    }
}


Result gemv_q4_mlx_simd(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                        const TesslQuantShape &shape, uint32_t layout, const TesslBuf *resid, OutKind out)
{
    const char *entry = resid ? "gemv_q4_mlx_simd_add" : "gemv_q4_mlx_simd";
    const bool staged = layout == TESSL_Q4_B200_STAGED;
    TESSL_TRY(refuse_layout(layout, entry, true));
    TESSL_TRY(bank_validate_layout(bank, shape, layout, entry));
    TESSL_TRY(require(x_bf16, shape.cols, 2, std::string(entry) + " x_bf16"));
    TESSL_TRY(require(y, shape.rows, out == OUT_BF16 ? 2 : 4, std::string(entry) + " y"));
    if (resid) TESSL_TRY(require(*resid, shape.rows, 4, std::string(entry) + " resid"));
    if (shape.rows == 0) return ok();
    const Named writes[] = {{"y", &y}};
    const Named reads[] = {{"packed", &bank.packed}, {"scales_biases", &bank.scales_biases}, {"x_bf16", &x_bf16}};
    TESSL_TRY(require_disjoint_writes(entry, writes, 1, reads, 3));
    if (!staged) TESSL_TRY(check_alignment(bank, entry));
    TESSL_TRY(require_aligned16(x_bf16, std::string(entry) + " x_bf16"));
    if (shape.cols == 0) {
        // No columns: every sum is empty. The kernel's loop never runs and the
        // epilogue stores 0 (+ resid), as the reference's does.
    }
    Q4GemvParams p{};
    p.seg[0] = make_seg(bank, nullptr, y, resid, shape.rows);
    p.nseg = 1;
    p.x = static_cast<const uint16_t *>(x_bf16.ptr);
    p.cols = shape.cols;
    p.group_shift = log2_u32(shape.group_size);
    p.epi = resid ? EPI_ADD_RESID : EPI_STORE;
    p.out_bf16 = out == OUT_BF16;
    p.staged = staged;
    return launch_q4_gemv(rt, p, 1, 1);
}

Result gemv_q4_mlx_gate_up(TesslRuntime *rt, const char *entry, const char *what, bool silu,
                           const TesslQ4MlxBank &gate, const TesslQ4MlxBank &up, const TesslBuf &x,
                           const TesslBuf &mid, const TesslQuantShape &shape, uint32_t layout, bool mid_as_bf16)
{
    const bool staged = layout == TESSL_Q4_B200_STAGED;
    TESSL_TRY(refuse_layout(layout, entry, true));
    TESSL_TRY(bank_validate_layout(gate, shape, layout, std::string(entry) + " gate"));
    TESSL_TRY(bank_validate_layout(up, shape, layout, std::string(entry) + " up"));
    TESSL_TRY(require(x, shape.cols, 2, std::string(entry) + " x"));
    if (mid_as_bf16) {
        TESSL_TRY(require(mid, shape.rows, 2, std::string(entry) + " mid (bf16)"));
    } else {
        TESSL_TRY(require(mid, shape.rows, 4, std::string(entry) + " mid"));
    }
    if (shape.rows == 0) return ok();
    const Named writes[] = {{"mid", &mid}};
    const Named reads[] = {{"gate_packed", &gate.packed},
                           {"gate_scales_biases", &gate.scales_biases},
                           {"up_packed", &up.packed},
                           {"up_scales_biases", &up.scales_biases},
                           {"x", &x}};
    TESSL_TRY(require_disjoint_writes(what, writes, 1, reads, 5));
    if (!staged) {
        TESSL_TRY(check_alignment(gate, std::string(entry) + " gate"));
        TESSL_TRY(check_alignment(up, std::string(entry) + " up"));
    }
    TESSL_TRY(require_aligned16(x, std::string(entry) + " x"));
    Q4GemvParams p{};
    p.staged = staged;
    p.seg[0] = make_seg(gate, &up, mid, nullptr, shape.rows);
    p.nseg = 1;
    p.x = static_cast<const uint16_t *>(x.ptr);
    p.cols = shape.cols;
    p.group_shift = log2_u32(shape.group_size);
    p.epi = silu ? EPI_GATE_UP_SILU : EPI_GATE_UP_GELU;
    p.out_bf16 = mid_as_bf16;
    return launch_q4_gemv(rt, p, 1, 2);
}

/// This rank's slot of its own gather buffer, as the output buffer of a sharded launch.
static Result sharded_out(const TesslPeerGather &g, const char *entry, uint64_t need_bytes, TesslBuf *out)
{
    TESSL_TRY(peer_gather_validate(g, entry));
    if (need_bytes > g.bytes_per_rank)
        return fmt("%s: the slice needs %llu bytes, the gather holds %llu per rank", entry, (unsigned long long)need_bytes,
                   (unsigned long long)g.bytes_per_rank);
    out->ptr = static_cast<uint8_t *>(g.buffers[g.rank]) + (size_t)g.rank * g.bytes_per_rank;
    out->nbytes = g.bytes_per_rank;
    return ok();
}

Result gemv_q4_mlx_simd_sharded(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16,
                                const TesslPeerGather &gather, const TesslQuantShape &shape, bool y_as_bf16, bool defer)
{
    const char *entry = "gemv_q4_mlx_simd_sharded";
    TesslBuf y{};
    TESSL_TRY(sharded_out(gather, entry, (uint64_t)shape.rows * (y_as_bf16 ? 2 : 4), &y));
    if (shape.rows == 0) return fmt("%s: a rank with no rows takes part through tessl_peer_gather", entry);
    TESSL_TRY(q4_bank_validate(bank, shape, entry));
    TESSL_TRY(require(x_bf16, shape.cols, 2, std::string(entry) + " x_bf16"));
    const Named writes[] = {{"gather slot", &y}};
    const Named reads[] = {{"packed", &bank.packed}, {"scales_biases", &bank.scales_biases}, {"x_bf16", &x_bf16}};
    TESSL_TRY(require_disjoint_writes(entry, writes, 1, reads, 3));
    TESSL_TRY(check_alignment(bank, entry));
    TESSL_TRY(require_aligned16(x_bf16, std::string(entry) + " x_bf16"));
    Q4GemvParams p{};
    p.seg[0] = make_seg(bank, nullptr, y, nullptr, shape.rows);
    p.nseg = 1;
    p.x = static_cast<const uint16_t *>(x_bf16.ptr);
    p.cols = shape.cols;
    p.group_shift = log2_u32(shape.group_size);
    p.epi = EPI_STORE;
    p.out_bf16 = y_as_bf16;
    p.peer = gather.world > 1 ? &gather : nullptr;
    p.peer_defer = defer;
    return launch_q4_gemv(rt, p, 1, 1);
}

Result gemv_q4_mlx_simd_gathered(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslPeerGather &gather,
                                 const TesslBuf &y, const TesslQuantShape &shape, const TesslBuf *resid, OutKind out)
{
    const char *entry = "gemv_q4_mlx_simd_gathered";
    TESSL_TRY(peer_gather_validate(gather, entry));
    TesslBuf x{};
    x.ptr = gather.buffers[gather.rank];
    x.nbytes = (uint64_t)gather.world * gather.bytes_per_rank;
    TESSL_TRY(q4_bank_validate(bank, shape, entry));
    TESSL_TRY(require(x, shape.cols, 2, std::string(entry) + " gathered x"));
    TESSL_TRY(require(y, shape.rows, out == OUT_BF16 ? 2 : 4, std::string(entry) + " y"));
    if (resid) TESSL_TRY(require(*resid, shape.rows, 4, std::string(entry) + " resid"));
    if (shape.rows == 0) return ok();
    const Named writes[] = {{"y", &y}};
    const Named reads[] = {{"packed", &bank.packed}, {"scales_biases", &bank.scales_biases}, {"gathered x", &x}};
    TESSL_TRY(require_disjoint_writes(entry, writes, 1, reads, 3));
    TESSL_TRY(check_alignment(bank, entry));
    Q4GemvParams p{};
    p.seg[0] = make_seg(bank, nullptr, y, resid, shape.rows);
    p.nseg = 1;
    p.x = static_cast<const uint16_t *>(x.ptr);
    p.cols = shape.cols;
    p.group_shift = log2_u32(shape.group_size);
    p.epi = resid ? EPI_ADD_RESID : EPI_STORE;
    p.out_bf16 = out == OUT_BF16;
    p.xwait = gather.world > 1 ? &gather : nullptr;
    return launch_q4_gemv(rt, p, 1, 1);
}

Result gemv_q4_mlx_gate_up_silu_sharded(TesslRuntime *rt, const TesslQ4MlxBank &gate, const TesslQ4MlxBank &up,
                                        const TesslBuf &x, const TesslPeerGather &gather, const TesslQuantShape &shape,
                                        bool mid_as_bf16, bool defer)
{
    const char *entry = "gemv_q4_mlx_gate_up_silu_sharded";
    TesslBuf mid{};
    TESSL_TRY(sharded_out(gather, entry, (uint64_t)shape.rows * (mid_as_bf16 ? 2 : 4), &mid));
    if (shape.rows == 0) return fmt("%s: a rank with no rows takes part through tessl_peer_gather", entry);
    TESSL_TRY(q4_bank_validate(gate, shape, std::string(entry) + " gate"));
    TESSL_TRY(q4_bank_validate(up, shape, std::string(entry) + " up"));
    TESSL_TRY(require(x, shape.cols, 2, std::string(entry) + " x"));
    const Named writes[] = {{"gather slot", &mid}};
    const Named reads[] = {{"gate_packed", &gate.packed},
                           {"gate_scales_biases", &gate.scales_biases},
                           {"up_packed", &up.packed},
                           {"up_scales_biases", &up.scales_biases},
                           {"x", &x}};
    TESSL_TRY(require_disjoint_writes(entry, writes, 1, reads, 5));
    TESSL_TRY(check_alignment(gate, std::string(entry) + " gate"));
    TESSL_TRY(check_alignment(up, std::string(entry) + " up"));
    TESSL_TRY(require_aligned16(x, std::string(entry) + " x"));
    Q4GemvParams p{};
    p.seg[0] = make_seg(gate, &up, mid, nullptr, shape.rows);
    p.nseg = 1;
    p.x = static_cast<const uint16_t *>(x.ptr);
    p.cols = shape.cols;
    p.group_shift = log2_u32(shape.group_size);
    p.epi = EPI_GATE_UP_SILU;
    p.out_bf16 = mid_as_bf16;
    p.peer = gather.world > 1 ? &gather : nullptr;
    p.peer_defer = defer;
    return launch_q4_gemv(rt, p, 1, 2);
}

Result gemv_q4_mlx_kv(TesslRuntime *rt, const TesslQ4MlxBank &k, const TesslQ4MlxBank &v, const TesslBuf &x_bf16,
                      const TesslBuf &k_out, const TesslBuf &v_out, const TesslQuantShape &shape, uint32_t layout)
{
    const char *entry = "gemv_q4_mlx_simd_kv";
    TESSL_TRY(refuse_layout(layout, entry));
    TESSL_TRY(q4_bank_validate(k, shape, std::string(entry) + " k"));
    TESSL_TRY(q4_bank_validate(v, shape, std::string(entry) + " v"));
    TESSL_TRY(require(x_bf16, shape.cols, 2, std::string(entry) + " x_bf16"));
    TESSL_TRY(require(k_out, shape.rows, 4, std::string(entry) + " k_out"));
    TESSL_TRY(require(v_out, shape.rows, 4, std::string(entry) + " v_out"));
    if (shape.rows == 0) return ok();
    const Named writes[] = {{"k_out", &k_out}, {"v_out", &v_out}};
    const Named reads[] = {{"k_packed", &k.packed},
                           {"k_scales_biases", &k.scales_biases},
                           {"v_packed", &v.packed},
                           {"v_scales_biases", &v.scales_biases},
                           {"x_bf16", &x_bf16}};
    TESSL_TRY(require_disjoint_writes("gemv_q4_mlx_kv", writes, 2, reads, 5));
    TESSL_TRY(check_alignment(k, std::string(entry) + " k"));
    TESSL_TRY(check_alignment(v, std::string(entry) + " v"));
    TESSL_TRY(require_aligned16(x_bf16, std::string(entry) + " x_bf16"));
    Q4GemvParams p{};
    p.seg[0] = make_seg(k, nullptr, k_out, nullptr, shape.rows);
    p.seg[1] = make_seg(v, nullptr, v_out, nullptr, shape.rows);
    p.nseg = 2;
    p.x = static_cast<const uint16_t *>(x_bf16.ptr);
    p.cols = shape.cols;
    p.group_shift = log2_u32(shape.group_size);
    p.epi = EPI_STORE;
    return launch_q4_gemv(rt, p, 1, 1);
}

Result gemv_q4_mlx_qkv(TesslRuntime *rt, const TesslQ4MlxBank &q, const TesslQ4MlxBank &k, const TesslQ4MlxBank &v,
                       const TesslBuf &x_bf16, const TesslQkvOutputs &out, uint32_t rows_q, uint32_t rows_kv,
                       uint32_t cols, uint32_t group_size, uint32_t layout)
{
    const char *entry = "gemv_q4_mlx_simd_qkv";
    TESSL_TRY(refuse_layout(layout, entry));
    const TesslQuantShape q_shape{rows_q, cols, group_size}, kv_shape{rows_kv, cols, group_size};
    TESSL_TRY(q4_bank_validate(q, q_shape, std::string(entry) + " q"));
    TESSL_TRY(q4_bank_validate(k, kv_shape, std::string(entry) + " k"));
    TESSL_TRY(q4_bank_validate(v, kv_shape, std::string(entry) + " v"));
    TESSL_TRY(require(x_bf16, cols, 2, std::string(entry) + " x_bf16"));
    TESSL_TRY(require(out.q_out, rows_q, 4, std::string(entry) + " q_out"));
    TESSL_TRY(require(out.k_out, rows_kv, 4, std::string(entry) + " k_out"));
    TESSL_TRY(require(out.v_out, rows_kv, 4, std::string(entry) + " v_out"));
    if (rows_q == 0 && rows_kv == 0) return ok();
    // Only the banks that produce output take part in the aliasing check.
    Named writes[3];
    Named reads[7];
    int nw = 0, nr = 0;
    if (rows_q != 0) {
        writes[nw++] = {"q_out", &out.q_out};
        reads[nr++] = {"q_packed", &q.packed};
        reads[nr++] = {"q_scales_biases", &q.scales_biases};
    }
    if (rows_kv != 0) {
        writes[nw++] = {"k_out", &out.k_out};
        writes[nw++] = {"v_out", &out.v_out};
        reads[nr++] = {"k_packed", &k.packed};
        reads[nr++] = {"k_scales_biases", &k.scales_biases};
        reads[nr++] = {"v_packed", &v.packed};
        reads[nr++] = {"v_scales_biases", &v.scales_biases};
    }
    reads[nr++] = {"x_bf16", &x_bf16};
    TESSL_TRY(require_disjoint_writes(entry, writes, nw, reads, nr));
    TESSL_TRY(require_aligned16(x_bf16, std::string(entry) + " x_bf16"));
    Q4GemvParams p{};
    p.nseg = 0;
    if (rows_q != 0) {
        TESSL_TRY(check_alignment(q, std::string(entry) + " q"));
        p.seg[p.nseg++] = make_seg(q, nullptr, out.q_out, nullptr, rows_q);
    }
    if (rows_kv != 0) {
        TESSL_TRY(check_alignment(k, std::string(entry) + " k"));
        TESSL_TRY(check_alignment(v, std::string(entry) + " v"));
        p.seg[p.nseg++] = make_seg(k, nullptr, out.k_out, nullptr, rows_kv);
        p.seg[p.nseg++] = make_seg(v, nullptr, out.v_out, nullptr, rows_kv);
    }
    p.x = static_cast<const uint16_t *>(x_bf16.ptr);
    p.cols = cols;
    p.group_shift = log2_u32(group_size);
    p.epi = EPI_STORE;
    return launch_q4_gemv(rt, p, 1, 1);
}

Result swiglu(TesslRuntime *rt, const TesslBuf &gate, const TesslBuf &up, const TesslBuf &out, uint32_t n,
              bool out_as_bf16)
{
    TESSL_TRY(require(gate, n, 4, "swiglu gate"));
    TESSL_TRY(require(up, n, 4, "swiglu up"));
    TESSL_TRY(require(out, n, out_as_bf16 ? 2 : 4, "swiglu out"));
    if (n == 0) return ok();
    swiglu_kernel<<<(n + 255) / 256, 256, 0, rt->stream>>>(static_cast<const float *>(gate.ptr),
                                                          static_cast<const float *>(up.ptr), out.ptr, n,
                                                          out_as_bf16 ? 1 : 0, 0);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "swiglu launch");
}

/// A validated prefill call with few rows, run as batches of up to 8 rows on the tensor-core GEMV kernel:
/// up to 24 rows that is faster than the prefill GEMM, whose 256-row tile would be mostly padding
/// (12288 x 4096: 9.3 us per batch of 8 against 34.6 us for any m <= 64). `*handled` is false when the shape
/// is not one that kernel is built for.
Result prefill_as_small_batches(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                                const TesslQuantShape &shape, uint32_t m, OutKind out, bool *handled)
{
    *handled = false;
    if (m == 0 || m > 24) return ok();
    Q4GemvParams probe{};
    probe.nseg = 1;
    probe.seg[0] = make_seg(bank, nullptr, y, nullptr, shape.rows);
    probe.cols = shape.cols;
    probe.group_shift = log2_u32(shape.group_size);
    if (!mma_ok(probe)) return ok();
    *handled = true;
    const size_t esz = out == OUT_BF16 ? 2 : 4;
    for (uint32_t b = 0; b < m; b += 8) {
        const uint32_t mb = std::min<uint32_t>(8u, m - b);
        Q4GemvParams p = probe;
        p.seg[0].out = static_cast<char *>(y.ptr) + (size_t)b * shape.rows * esz;
        p.x = static_cast<const uint16_t *>(x_bf16.ptr) + (size_t)b * shape.cols;
        p.epi = EPI_STORE;
        p.out_bf16 = out == OUT_BF16;
        TESSL_TRY(launch_q4_gemv(rt, p, (int)mb, 1));
    }
    return ok();
}

Result gemm_q4_mlx(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                   const TesslQuantShape &shape, uint32_t m, uint32_t layout, const TesslBuf *resid, OutKind out)
{
    const char *entry = resid ? "gemm_q4_mlx_simd_add" : "gemm_q4_mlx_simd";
    TESSL_TRY(refuse_layout(layout, entry));
    if (m == 0) return ok();
    if (m > TESSL_GEMM_Q4_MLX_MAX_M) {
        return fmt("%s: M = %u exceeds GEMM_MAX_M = %u; the kernel clamps to that internally, so rows %u..%u would "
                   "be left unwritten rather than computed",
                   entry, m, TESSL_GEMM_Q4_MLX_MAX_M, TESSL_GEMM_Q4_MLX_MAX_M, m);
    }
    TESSL_TRY(q4_bank_validate(bank, shape, entry));
    const uint64_t out_elems = elems(m, shape.rows);
    TESSL_TRY(require(x_bf16, elems(m, shape.cols), 2, std::string(entry) + " x_bf16"));
    TESSL_TRY(require(y, out_elems, out == OUT_BF16 ? 2 : 4, std::string(entry) + " y"));
    if (resid) TESSL_TRY(require(*resid, out_elems, 4, std::string(entry) + " resid"));
    if (shape.rows == 0) return ok();
    const Named writes[] = {{"y", &y}};
    const Named reads[] = {{"packed", &bank.packed}, {"scales_biases", &bank.scales_biases}, {"x_bf16", &x_bf16}};
    TESSL_TRY(require_disjoint_writes("gemm_q4_mlx", writes, 1, reads, 3));
    TESSL_TRY(check_alignment(bank, entry));
    TESSL_TRY(require_aligned16(x_bf16, std::string(entry) + " x_bf16"));
    Q4GemvParams p{};
    p.seg[0] = make_seg(bank, nullptr, y, resid, shape.rows);
    p.nseg = 1;
    p.x = static_cast<const uint16_t *>(x_bf16.ptr);
    p.cols = shape.cols;
    p.group_shift = log2_u32(shape.group_size);
    p.epi = resid ? EPI_ADD_RESID : EPI_STORE;
    p.out_bf16 = out == OUT_BF16;
    return launch_q4_gemv(rt, p, (int)m, 1);
}

Result embed_lookup_q4_mlx(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &token_ids, const TesslBuf &out,
                           uint32_t vocab, uint32_t hidden, uint32_t group_size, uint32_t n_tokens)
{
    const char *what = "embed_lookup_q4_mlx";
    const TesslQuantShape shape{vocab, hidden, group_size};
    TESSL_TRY(q4_bank_validate(bank, shape, what));
    const uint64_t total = elems(n_tokens, hidden);
    TESSL_TRY(require(token_ids, n_tokens, 4, std::string(what) + " token_ids"));
    TESSL_TRY(require(out, total, 4, std::string(what) + " out"));
    const Named writes[] = {{"out", &out}};
    const Named reads[] = {{"packed", &bank.packed}, {"scales_biases", &bank.scales_biases}, {"token_ids", &token_ids}};
    TESSL_TRY(require_disjoint_writes(what, writes, 1, reads, 3));
    if (total == 0) return ok();
    TESSL_TRY(check_alignment(bank, what));
    TESSL_TRY(require_aligned16(out, std::string(what) + " out"));
    if (((uintptr_t)token_ids.ptr & 3u) != 0) return fmt("%s token_ids: device pointer must be 4-byte aligned", what);
    const uint64_t total32 = total / 32;  // hidden is a multiple of the group size, itself a multiple of 32
    embed_lookup_q4_mlx_kernel<<<(unsigned)((total32 + 127) / 128), 128, 0, rt->stream>>>(
        static_cast<const uint8_t *>(bank.packed.ptr), static_cast<const uint32_t *>(bank.scales_biases.ptr),
        static_cast<const uint32_t *>(token_ids.ptr), static_cast<float *>(out.ptr), hidden, log2_u32(group_size), vocab,
        total32);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "embed_lookup_q4_mlx launch");
}

uint64_t q4_mlx_staged_bytes(uint32_t rows, uint32_t cols, uint32_t group_size)
{
    if (!staged_domain(cols, group_size)) return 0;
    return (uint64_t)((rows + 7) / 8) * staged_geom(cols, group_size).unit_bytes;
}

Result q4_mlx_repack_staged(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslQuantShape &shape, const TesslBuf &out)
{
    const char *entry = "q4_mlx_repack_staged";
    TESSL_TRY(q4_bank_validate(bank, shape, entry));
    if (!staged_domain(shape.cols, shape.group_size))
        return fmt("%s: the B200 staged layout exists for rows of 1024, 2048 or 4096 columns and groups of 32, 64 or 128 "
                   "(got %u columns, group %u)", entry, shape.cols, shape.group_size);
    const uint64_t nbytes = q4_mlx_staged_bytes(shape.rows, shape.cols, shape.group_size);
    TESSL_TRY(require(out, nbytes, 1, std::string(entry) + " out"));
    if (shape.rows == 0) return ok();
    const Named writes[] = {{"out", &out}};
    const Named reads[] = {{"packed", &bank.packed}, {"scales_biases", &bank.scales_biases}};
    TESSL_TRY(require_disjoint_writes(entry, writes, 1, reads, 2));
    TESSL_TRY(require_aligned16(bank.packed, std::string(entry) + " packed"));
    TESSL_TRY(require_aligned16(bank.scales_biases, std::string(entry) + " scales_biases"));
    TESSL_TRY(require_aligned16(out, std::string(entry) + " out"));
    const uint64_t n16 = nbytes / 16;
    q4_repack_staged_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, rt->stream>>>(
        static_cast<const uint4 *>(bank.packed.ptr), static_cast<const uint4 *>(bank.scales_biases.ptr),
        static_cast<uint4 *>(out.ptr), shape.rows, shape.cols, shape.group_size, n16);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "q4_mlx_repack_staged launch");
}

Result q4_mlx_unpack(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslQuantShape &shape, const TesslBuf &out)
{
    TESSL_TRY(q4_bank_validate(bank, shape, "q4_mlx_unpack"));
    const uint64_t n = elems(shape.rows, shape.cols);
    TESSL_TRY(require(out, n, 1, "q4_mlx_unpack out"));
    if (n == 0) return ok();
    const uint64_t bytes = n / 2;
    q4_unpack_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, rt->stream>>>(
        static_cast<const uint8_t *>(bank.packed.ptr), static_cast<uint8_t *>(out.ptr), bytes);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "q4_mlx_unpack launch");
}

Result q4_mlx_dequant(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslQuantShape &shape,
                      const TesslBuf &out)
{
    TESSL_TRY(q4_bank_validate(bank, shape, "q4_mlx_dequant"));
    const uint64_t n = elems(shape.rows, shape.cols);
    TESSL_TRY(require(out, n, 4, "q4_mlx_dequant out"));
    if (n == 0) return ok();
    const uint64_t bytes = n / 2;
    q4_dequant_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, rt->stream>>>(
        static_cast<const uint8_t *>(bank.packed.ptr), static_cast<const uint32_t *>(bank.scales_biases.ptr),
        static_cast<float *>(out.ptr), shape.rows, shape.cols, log2_u32(shape.group_size));
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "q4_mlx_dequant launch");
}

}  // namespace nn
}  // namespace tessl
