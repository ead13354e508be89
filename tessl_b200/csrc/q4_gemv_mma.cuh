// Q4 GEMV / small-batch GEMM (M <= 8, rows of 1024, 2048 or 4096 columns; one row of x also over rows of 8192 and
// 12288 columns) and MLX-layout Q8 (M <= 8), with the dot products on the tensor cores.
//
// Why: on the FMA pipe a weight costs one FMA plus 7/8 of a bit-manipulation
// instruction plus overheads, about 2 issue slots; HBM3e delivers ~46 weights
// per clock and SM, which would need ~90 of the SM's 128 slots per clock, and
// the FMA-pipe kernels measured compute-bound at ~30 weights per clock (73% of
// the memory roofline on a long stream). A nibble pair masked in place is
// already the register layout of an `mma.sync.m16n8k16` A fragment: read as bf16
// bit patterns, 0..15 and 16 x (0..15) are q * 2^-133 exactly (the subnormals and
// the first binade are one linear scale), and the activations carry the rest
// (scaled by a power of two, the partners of the odd nibbles by a sixteenth of it).
// So one MMA replaces 256 FMAs: 16 weight rows x 16 columns against the
// activations as the B operand, whose 8 columns are the up to 8 rows of the batch
// (for M = 1 all 8 hold the same vector). The kernel is then bound by the weight
// stream on a long launch and by its start and the consumers' ALU rate on a short one.
//
// Structure (one persistent block per SM, 18 warps):
//   warp 16   producer: sets up the barriers, then streams row blocks (16 rows of one
//             bank, or 8 + 8 rows of a gate/up pair) through a ring of stages with plain
//             `cp.async.bulk` copies, one per PAIR of adjacent rows or per four rows (each
//             issued by its own lane): the copy engine's cost is per copy more than per
//             byte (sixteen 2 KB copies per stage held a long stream to 0.75 of the HBM
//             rate, eight 4 KB copies reach 0.9, four 8 KB copies the pure read rate). The
//             pairs sit 32 bytes past a multiple of 128 apart (bank-conflict-free reads),
//             and the two rows of a pair are the MMA rows g and g + 8 that one lane group
//             reads. Plus the rows' scale/bias pairs. It never waits for the preceding
//             kernel (weights are not written by it) nor for the other warps of its block.
//   warps 0-15 consumers: warp w owns columns [w K/16, (w+1) K/16) of every row (of every
//             4096-column window of a long row). After the dependency wait it stages its
//             slice of x once; the B fragments then stay in registers for the whole launch
//             (long rows: reloaded from the staged copy per window). Per stage it runs one
//             MMA chain per quantization group (the chain starts from zero because each
//             group has its own scale), folds `scale * dot + bias * xsum` in f32 like the
//             reference's qdot16, and leaves its partial sums in shared memory.
//   warp 17   reducer: adds the 16 partial sums of each output in warp order, applies the
//             epilogue (residual, SiLU/GELU gate) and stores - in a column-sharded launch
//             also into every peer GPU's gather buffer, followed by the flag exchange.
// A row's summation order depends only on K and the group size, so fused
// gate/up, K/V and Q/K/V launches give the same bits as separate launches.
//
// Every mbarrier wait and every wait for a peer is bounded (see q4_gemv_tma.cuh).
#pragma once
#include <cstddef>

#include "q4_gemv_tma.cuh"

namespace tessl {
namespace q4m {

using q4k::bulk_g2s;
using q4k::lds32;
using q4k::mbar_arrive;
using q4k::mbar_expect_tx;
using q4k::mbar_init;
using q4k::mbar_try;
using q4k::mbar_wait;
using q4k::smem_u32;

// Blocks per SM the register budget is compiled for (2 lets the next launch's block start
// beside this one's when the ring is short enough).
#ifndef TESSL_GEMV_MMA_MIN_BLOCKS
#define TESSL_GEMV_MMA_MIN_BLOCKS 1
#endif
constexpr int kConsumers = 16;
constexpr int kThreads = (kConsumers + 2) * 32;
constexpr uint32_t kHoldFrom = 3, kHoldMaxStages = 16;  // see the producer loop
constexpr uint32_t kRowPad = 32;  // bytes; row pitch = K / 2 + 32
constexpr uint32_t kXStageBytes = 512 + 32;  // a warp's staged slice of x: B fragments and up to 8 group sums

struct Seg {
    const uint8_t *packed0;
    const uint32_t *sb0;
    const uint8_t *packed1;  // second bank of a gate/up launch
    const uint32_t *sb1;
    void *out;
    const float *resid;
    uint32_t rows;
    uint32_t rb_begin;  // first row block of this bank within the launch
};

/// Exchange of a column-sharded launch's outputs over NVLink peer memory (world <= 1: none). The
/// flag words are those of peer_gather.cu: [0, 8) arrivals by source rank, [8, 16) completions by
/// source rank, [16] this rank's call counter, [17] the ticket counter of the call's blocks.
struct Peer {
    uint8_t *out[8];     // where seg[0].out of THIS rank lives in rank r's gather buffer (out[rank] == seg[0].out)
    uint32_t *flags[8];  // flag words of every rank
    uint32_t rank, world;
    long long wait_clocks;  // bound of every wait for a peer
    // 1: the launch tells its peers that its outputs are complete but does not wait for theirs; the kernel that
    // reads the gathered vector does (`XWait`), behind its own weight prefetch.
    uint32_t defer;
};

/// The activations are a gather buffer whose last exchange was launched with `defer`: before reading x, wait
/// until every peer's completion flag has reached this rank's call counter (world <= 1: nothing to wait for).
struct XWait {
    const uint32_t *flags;  // this rank's flag words
    uint32_t rank, world;
    long long wait_clocks;
};

/// Field order: what a launch without an exchange reads before its first copy and its first MMA sits in the first
/// two 64-byte lines of the parameter block (the constant cache is cold for every launch); worth 0.02-0.04 us per
/// launch when measured, so a tidiness more than an optimisation.
struct Params {
    // --- line 0: the scalars every role reads
    uint32_t cols;
    uint32_t group_shift;
    uint32_t stages;
    uint32_t total_rb;
    int nseg;
    uint32_t m;
    int epi;
    int out_bf16;
    // A launch may cover a window of `cols` columns of longer rows (a K chunk): bytes between packed
    // rows and between scale/bias rows in global memory, elements between the batch rows of x. Dense
    // rows: cols / 2, (cols >> group_shift) * 4 and cols.
    uint32_t row_pitch;
    uint32_t sb_pitch;
    uint32_t x_pitch;
    uint32_t quads;  // fetch four rows per bulk copy (long streams, one bank, one row of x)
    // Row blocks per thread block as a 32.32 fixed-point number, rounded up: block b takes the row blocks
    // [b step >> 32, (b + 1) step >> 32) clipped to total_rb. (The division total_rb b / blocks in the kernel is a
    // 64-bit one, executed by all eighteen warps at once: ~900 issue cycles before the block's first copy.)
    uint32_t rb_step_lo, rb_step_hi;
    uint32_t peer_world;   // == peer.world
    uint32_t xwait_world;  // == xwait.world
    // --- line 1: the activations and the first bank
    const uint16_t *x;  // bf16 [m, cols]
    Seg seg[3];
    // --- cold: failure reports and the exchange
    uint32_t *status;
    Peer peer;
    XWait xwait;
};
static_assert(offsetof(Params, x) == 64 && offsetof(Params, seg) == 72 && sizeof(Seg) == 56, "parameter lines");

// A system-scope fence, and every acquire or release at system scope, costs ~1.8 us on this GPU (measured: the
// same for local and for peer stores). The exchange therefore polls and signals with RELAXED system-scope
// accesses and places the few fences it needs by hand, each where its latency is hidden or paid once.
__device__ __forceinline__ void st_relaxed_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

/// Lane t < world (t != rank) of the calling warp waits until flag word `base + t` of this rank (`mine`) reaches
/// `seq`; false (and a status word, role 0x50 like the stand-alone gather) when the bound runs out. The poll is
/// relaxed: a caller that goes on to READ what the flag announces inside the same kernel fences afterwards.
__device__ __forceinline__ bool peer_wait(const uint32_t *mine, uint32_t rank, uint32_t world, long long wait_clocks,
                                          uint32_t *status, uint32_t base, uint32_t seq, uint32_t code)
{
    const uint32_t lane = threadIdx.x & 31;
    bool ok_ = true;
    if (lane < world && lane != rank) {
        const uint32_t *f = mine + base + lane;
        const long long t0 = clock64();
        while ((int32_t)(ld_relaxed_sys(f) - seq) < 0) {
            if (clock64() - t0 > wait_clocks) {
                *(volatile uint32_t *)status = (0x50u << 24) | (code << 16) | lane;
                ok_ = false;
                break;
            }
            __nanosleep(64);
        }
    }
    return __all_sync(0xffffffffu, ok_);
}

__device__ __forceinline__ uint2 lds64(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/// SW: packed words a lane reads per row of its warp's slice (K / 512).
/// WPG: words of one lane per quantization group (G / 32).
/// NB: banks per row block (2 = gate/up: rows 0-7 of the MMA are gate rows, 8-15 the same rows of up).
/// BATCH: the 8 MMA columns are distinct batch rows (M >= 2) instead of 8 copies of one vector.
/// Q8: the rows hold 8-bit codes. A code c = 16 h + l is taken as its two nibbles l, h against the
///     activations x and 16 x (exact in bf16), so a row of K codes runs as a row of 2 K nibbles:
///     `cols` and the group size are given in nibbles (2 K, 2 G), x has cols / 2 elements per row.
/// NWIN: windows of 512 SW columns a row consists of (M = 1, one bank): rows of 8192 or 12288 columns run as
///     2 or 3 windows inside every stage, each warp taking its slice of every window in turn, so that a
///     long-row projection is still one launch with one fixed part.
/// ROWS: rows per stage (16, or 14 where two stages of 16 long rows would not fit in shared memory; the
///     MMA's unused rows cost nothing that matters: the kernel is bound by the weight stream).
/// STAGED: the banks are in the staged layout (a compile-time choice: as a run-time one its address arithmetic
///     cost the row-major launches 2-3 %).
template <int SW, int WPG, int NB, bool BATCH, bool Q8 = false, int NWIN = 1, int ROWS = 16, bool STAGED = false>
__global__ void __launch_bounds__(kThreads, TESSL_GEMV_MMA_MIN_BLOCKS) q4_gemv_mma_kernel(const Params p)
{
    static_assert(!STAGED || (NWIN == 1 && ROWS == 16 && !BATCH && !Q8), "staged banks: the one-row Q4 kernel");
    asm volatile("griddepcontrol.launch_dependents;");
    static_assert(NWIN == 1 || (NB == 1 && !BATCH && !Q8), "windows: one bank, one row of x, Q4");
    static_assert(ROWS % (2 * NB) == 0 && ROWS <= 16, "whole row pairs per bank");
    constexpr int NGS = SW / WPG;     // groups per slice
    constexpr int RPB = ROWS / NB;    // rows per bank and stage
    constexpr int NQ = (NGS + 3) / 4;  // affine groups per lane when M = 1
    static_assert(SW % WPG == 0 && NGS >= 1, "a warp's slice holds whole groups");
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t K = p.cols, gpr = K >> p.group_shift;
    const uint32_t row_bytes = K >> 1, pitch = row_bytes + kRowPad, sb_row_bytes = gpr * 4;
    // MMA rows g and g + 8 (both read by lane group g) are two ADJACENT rows of a bank, 2 l and 2 l + 1, kept
    // back to back in shared memory so that one bulk copy fetches both: the copy engine's cost is per
    // copy more than per byte, and sixteen 2 KB copies per stage bounded the stream. Pairs sit 32 bytes
    // past a multiple of 128 apart (bank-conflict-free fragment reads).
    const uint32_t pair_pitch = 2 * row_bytes + kRowPad;
    // `quads` (dense rows, one row of x): two pairs of a bank back to back so that one copy fetches four rows -
    // eight copies of 4 KB per stage still cost the copy unit more than the bytes do, four of 8 KB reach the
    // pure read rate on a long stream - with the quads 32 bytes past a multiple of 128 apart. The two pairs of
    // a quad then share banks (a two-way conflict on every fragment read), which the copies more than pay
    // for at every launch size measured. Pure data movement: results do not depend on it.
    const bool quads = !BATCH && p.quads != 0;
    constexpr bool staged = STAGED;
    const uint32_t unit_bytes = 4 * pair_pitch + 8 * sb_row_bytes;  // one staged unit: 8 rows
    auto pair_off = [&](uint32_t gi) {
        if (staged) return (gi >> 2) * unit_bytes + (gi & 3u) * pair_pitch;
        return quads ? (gi >> 1) * (4 * row_bytes + kRowPad) + (gi & 1u) * 2 * row_bytes : gi * pair_pitch;
    };
    const uint32_t part_bytes = BATCH ? kConsumers * 16 * 8 * 4 : kConsumers * 16 * 4;
    const uint32_t off_sb = (ROWS / 2) * 2 * pitch, off_part = off_sb + ROWS * sb_row_bytes;
    const uint32_t stage_bytes = off_part + part_bytes;
    // scale/bias rows of lane group gi's pair (local rows 2 gi and 2 gi + 1)
    auto sb_pair_off = [&](uint32_t gi) {
        if (staged) return (gi >> 2) * unit_bytes + 4 * pair_pitch + 2 * (gi & 3u) * sb_row_bytes;
        return off_sb + 2 * gi * sb_row_bytes;
    };
    const uint32_t S = p.stages;
    const uint32_t ring = smem_u32(smem);
    const uint32_t bars = ring + S * stage_bytes;
    auto full = [&](uint32_t s) { return bars + 8 * s; };
    auto empty = [&](uint32_t s) { return bars + 8 * (S + s); };
    auto done = [&](uint32_t s) { return bars + 8 * (2 * S + s); };
    // M = 1: each warp stages its slice of x once (512 bytes of B fragments + the group sums) and the
    // lanes read their fragments back, instead of every lane converting the 64 values it holds.
    const uint32_t xbar = bars + 24 * S;  // consumers: x is in registers (the producer holds the ring's tail for it)
    const uint32_t xstage = ((bars + 24 * S + 8 + 15u) & ~15u) + (uint32_t)warp * (kXStageBytes * NWIN);

    auto rb_at = [&](uint32_t b) {
        const uint32_t v = __umulhi(b, p.rb_step_lo) + b * p.rb_step_hi;
        return min(v, p.total_rb);
    };
    const uint32_t rb_lo = rb_at(blockIdx.x);
    const uint32_t n_local = rb_at(blockIdx.x + 1) - rb_lo;

    // The producer warp sets up the barriers and goes straight on to its first copies: it only ARRIVES at the
    // block's start barrier, the other warps wait there for that arrival. (With a __syncthreads() here the first
    // copy left 2600 cycles after the block's first instruction.)
    if (warp == kConsumers) {
        // one barrier per lane: full and empty (one arrival each), then done and xbar (one per consumer warp)
        if (lane == 0) abort_flag = 0;
        if ((uint32_t)lane <= 3 * S) mbar_init(bars + 8 * lane, (uint32_t)lane < 2 * S ? 1u : (uint32_t)kConsumers);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copies' completions see the barriers (0.02 us)
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"n"(kThreads) : "memory");
    } else {
        asm volatile("bar.sync 2, %0;" ::"n"(kThreads) : "memory");
    }
    volatile int *abortp = &abort_flag;
    auto fail = [&](uint32_t role, uint32_t where) {
        *abortp = 1;
        // the first report stands: warps that leave because another one gave up do not overwrite its reason
        if (*(volatile uint32_t *)p.status == 0)
            *(volatile uint32_t *)p.status = (0x40u << 24) | (role << 20) | (where & 0xfffffu);
    };
    auto locate = [&](uint32_t rb, Seg &sg, uint32_t &row0) {
        int s = 0;
        if (p.nseg > 1 && rb >= p.seg[1].rb_begin) s = 1;
        if (p.nseg > 2 && rb >= p.seg[2].rb_begin) s = 2;
        sg = p.seg[s];
        row0 = (rb - sg.rb_begin) * RPB;
    };

    if (warp == kConsumers) {
        // ------------------------------------------------ producer ---
        // The whole warp runs the loop; per stage lane 0 posts the byte count and each
        // row's copy is issued by its own lane (issuing them all from one thread costs
        // about as long as the copies take to arrive). The loop is kept to a handful of
        // instructions per stage: the warp shares its scheduler with consumer warps that
        // saturate it, so every instruction here waits for an issue slot. Lanes 0-15 own
        // the 16 row slots of a stage, lanes 16 (and 17) the scale/bias rows of a bank.
        // Windowed rows (NB = 1 only): the scale/bias rows are not contiguous, lanes 16-31 fetch one each.
        const bool sb_by_row = NB == 1 && p.sb_pitch != sb_row_bytes;
        const bool pair_copy = p.row_pitch == row_bytes;  // dense rows: two adjacent rows are one contiguous range
        constexpr uint32_t HP = RPB / 2;                  // row pairs per bank and stage
        // lane m < 16 owns MMA row m: lane group g = m % 8, upper half hi = m / 8 -> bank g / HP, local row 2 (g % HP) + hi
        const uint32_t mg = (uint32_t)lane & 7u, mhi = ((uint32_t)lane >> 3) & 1u;
        const uint32_t my_bank = lane < 16 ? mg / HP : (sb_by_row ? 0u : (uint32_t)lane - 16);
        const uint32_t my_r = lane < 16 ? 2 * (mg % HP) + mhi : (sb_by_row ? (uint32_t)lane - 16 : 0u);
        const bool copies = lane < 16 ? mg < HP * NB : (sb_by_row ? lane - 16 < RPB : lane < 16 + NB);
        const uint32_t my_dst = lane < 16 ? pair_off(mg) + mhi * row_bytes
                                          : off_sb + (sb_by_row ? my_r : my_bank * RPB) * sb_row_bytes;
        uint32_t s = 0, ph = 0, issued = 0;
        // the first stage that waits for x (see the loop); a block of exactly three stages holds its last one
        // (6144 x 4096: 4.64 -> 4.47 us)
        const uint32_t hold_from = NWIN > 1 ? 1u : (n_local == 3 ? 2u : kHoldFrom);
        int cur_seg = -1;
        uint32_t seg_end_rb = 0, seg_rows = 0, row0 = 0;
        const uint8_t *src = nullptr;   // this lane's next source: a packed row (lanes 0-15) or the block's scale rows
        uint32_t src_step = 0;
        for (uint32_t j = 0; j < n_local; ++j) {
            const uint32_t rb = rb_lo + j;
            if (cur_seg < 0 || rb >= seg_end_rb) {
                // entering a bank: this lane's source pointer and stride within it
                int sidx = 0;
                if (p.nseg > 1 && rb >= p.seg[1].rb_begin) sidx = 1;
                if (p.nseg > 2 && rb >= p.seg[2].rb_begin) sidx = 2;
                cur_seg = sidx;
                const Seg &sg = p.seg[sidx];
                seg_rows = sg.rows;
                seg_end_rb = sg.rb_begin + (sg.rows + RPB - 1) / RPB;
                row0 = (rb - sg.rb_begin) * RPB;
                if (lane < 16) {
                    src = (my_bank == 0 ? sg.packed0 : sg.packed1) + (size_t)(row0 + my_r) * p.row_pitch;
                    src_step = RPB * p.row_pitch;
                } else {
                    src = reinterpret_cast<const uint8_t *>((my_bank == 0 ? sg.sb0 : sg.sb1)) +
                          (size_t)(row0 + (sb_by_row ? my_r : 0u)) * p.sb_pitch;
                    src_step = RPB * p.sb_pitch;
                }
            }
            if (!mbar_wait(empty(s), ph ^ 1u, abortp, 64)) {
                if (lane == 0) fail(1, j);
                break;
            }
            // A short launch asks for three stages of its ring at once (one, where a stage holds rows of 8192 or 12288
            // columns) and for the rest once the consumers hold x. Every block's whole ring requested at the block's
            // start has two costs: the load of x, issued when the previous launch has ended, returns behind whatever
            // copies this SM still has in flight, and the first stage of a block that starts late waits behind the
            // other blocks' later stages. 12288 x 4096 back to back: 7.9 -> 7.2 us, 18992 x 4096 10.0 -> 9.6 us,
            // 4096 x 12288 8.3 -> 7.8 us; a long stream loses the idle start instead (151936 x 4096: 52.4 -> 52.8 us),
            // hence the limit. Releasing the tail earlier (at the dependency wait's return, or once x is in registers)
            // gave 7.2 us where this gives 6.8; two or four stages instead of three were slower (also for Q8, whose
            // stages are larger: a rule by bytes in flight does not describe it); letting the blocks with the most
            // stages skip the hold changed nothing.
            if (j == hold_from && n_local <= kHoldMaxStages && !mbar_wait(xbar, 0, abortp, 64)) {
                if (lane == 0) fail(1, j);
                break;
            }
            const uint32_t nrows = min((uint32_t)RPB, seg_rows - row0);
            const uint32_t st = ring + s * stage_bytes;
            if constexpr (STAGED) {
                // one bank: units 2 b and 2 b + 1 of the block; a gate/up pair: unit b of each bank
                const Seg &sg = p.seg[cur_seg];
                const uint32_t ua = row0 / 8, ub = NB == 1 ? ua + 1 : ua;
                const bool has_b = NB == 2 || ub < (seg_rows + 7) / 8;
                if (lane == 0) mbar_expect_tx(full(s), (has_b ? 2u : 1u) * unit_bytes);
                __syncwarp();
                if (lane == 0) bulk_g2s(st, sg.packed0 + (size_t)ua * unit_bytes, unit_bytes, full(s));
                if (lane == 1 && has_b)
                    bulk_g2s(st + unit_bytes, (NB == 1 ? sg.packed0 : sg.packed1) + (size_t)ub * unit_bytes, unit_bytes, full(s));
                row0 += RPB;
                ++issued;
                if (++s == S) s = 0, ph ^= 1u;
                continue;
            }
            if (lane == 0) mbar_expect_tx(full(s), NB * nrows * (row_bytes + sb_row_bytes));
            __syncwarp();
            if (copies) {
                if (lane >= 16) {
                    if (!sb_by_row) {
                        bulk_g2s(st + my_dst, src, nrows * sb_row_bytes, full(s));
                    } else if (my_r < nrows) {
                        bulk_g2s(st + my_dst, src, sb_row_bytes, full(s));
                    }
                } else if (pair_copy) {
                    if (quads && nrows == RPB) {
                        if (mhi == 0 && (mg & 1u) == 0 && mg < HP * NB)
                            bulk_g2s(st + my_dst, src, ((mg % HP) + 1 < HP ? 4 : 2) * row_bytes, full(s));
                    } else if (mhi == 0 && my_r < nrows) bulk_g2s(st + my_dst, src, my_r + 1 < nrows ? 2 * row_bytes : row_bytes, full(s));
                } else if (my_r < nrows) {
                    bulk_g2s(st + my_dst, src, row_bytes, full(s));
                }
            }
            src += src_step, row0 += RPB;
            ++issued;
            if (++s == S) s = 0, ph ^= 1u;
        }
        // After a timeout elsewhere copies may still be in flight: give the last ring a bounded chance to land.
        if (*abortp && lane == 0) {
            for (uint32_t i = issued > S ? issued - S : 0; i < issued; ++i) {
                const long long t0 = clock64();
                while (!mbar_try(full(i % S), (i / S) & 1u))
                    if (clock64() - t0 > 4000000000ll) break;
            }
        }
    } else if (warp == kConsumers + 1) {
        // ------------------------------------------------ reducer ---
        asm volatile("griddepcontrol.wait;" ::: "memory");  // y and resid belong to the stream's order
        // Sharded launch: the outputs also go to every peer's gather buffer, so this kernel is the
        // exchange. Arrival first - this rank's earlier readers of its buffer precede this kernel in
        // stream order, so "I am here" tells the peers they may overwrite it - then the stores as rows
        // finish, then one completion handshake by the block that finishes last. The arrival round trip
        // hides behind the weight stream; only the completion one is exposed.
        const bool peered = !BATCH && p.peer_world > 1;
        uint32_t seq = 0;
        bool good = true;
        if (peered) {
            seq = *(volatile uint32_t *)(p.peer.flags[p.peer.rank] + 16) + 1;  // advanced by the call's last block only
            if (blockIdx.x == 0 && (uint32_t)lane < p.peer.world && (uint32_t)lane != p.peer.rank)
                st_relaxed_sys(p.peer.flags[lane] + p.peer.rank, seq);  // announces no data: the earlier readers of this
                                                                        // rank's buffer finished before this kernel began
            if (!peer_wait(p.peer.flags[p.peer.rank], p.peer.rank, p.peer.world, p.peer.wait_clocks, p.status, 0, seq, 3))
                *abortp = 1, good = false;
        }
        uint32_t s = 0, ph = 0;
        for (uint32_t j = 0; good && j < n_local; ++j) {
            // where the stage's outputs go, looked up while the consumers are still at work on it
            Seg sg;
            uint32_t row0;
            locate(rb_lo + j, sg, row0);
            const float rv = (p.epi == q4k::EPI_ADD_RESID && !BATCH && lane < RPB && row0 + lane < sg.rows) ? sg.resid[row0 + lane] : 0.0f;
            if (!mbar_wait(done(s), ph, abortp, 32)) {
                if (lane == 0) fail(3, j);
                good = false;
                break;
            }
            const uint32_t part = ring + s * stage_bytes + off_part;
            if constexpr (!BATCH) {
                // lane r < RPB: output row row0 + r (for a gate/up pair also its up partner, MMA row r + 8)
                const bool live = lane < RPB && row0 + lane < sg.rows;
                const uint32_t row = row0 + lane;
                float v = 0.0f;
                if (live) {
                    float v0 = 0.0f, v1 = 0.0f;
                    // local row l sits in MMA row (l odd ? 8 : 0) + l / 2; its up partner RPB / 2 rows further
                    const uint32_t mrow = (((uint32_t)lane & 1u) << 3) + ((uint32_t)lane >> 1);
#pragma unroll
                    for (int w = 0; w < kConsumers; ++w) {
                        v0 += __uint_as_float(lds32(part + (w * 16 + mrow) * 4));
                        if (NB == 2) v1 += __uint_as_float(lds32(part + (w * 16 + mrow + RPB / 2) * 4));
                    }
                    v = v0;
                    if (p.epi == q4k::EPI_ADD_RESID) {
                        v = v + rv;
                    } else if (p.epi == q4k::EPI_GATE_UP_SILU) {
                        v = dev::silu(v0) * v1;
                    } else if (p.epi == q4k::EPI_GATE_UP_GELU) {
                        v = dev::gelu_pytorch_tanh(v0) * v1;
                    }
                }
                // The partial sums are in registers: the stage may be refilled while the outputs are stored (stores to
                // a peer GPU take their time, and the producer waits for this arrival).
                __syncwarp();
                if (lane == 0) mbar_arrive(empty(s));
                const uint32_t hbits = p.out_bf16 ? (uint32_t)dev::f32_to_bf16_store(v) : __float_as_uint(v);
                if (live) {
                    if (p.out_bf16) {
                        static_cast<uint16_t *>(sg.out)[row] = (uint16_t)hbits;
                    } else {
                        static_cast<float *>(sg.out)[row] = v;
                    }
                }
                if (peered) {
                    if (row0 + RPB <= sg.rows) {
                        // A whole block: every lane collects the block's outputs, and lane L stores them to peer L with
                        // 16-byte stores - one or a few store instructions per stage for all peers together, where a
                        // store per row and peer made the reducer the slowest part of a sharded launch.
                        const bool to_peer = (uint32_t)lane < p.peer.world && (uint32_t)lane != p.peer.rank;
                        if (p.out_bf16) {
                            const uint32_t word = (hbits & 0xffffu) | (__shfl_down_sync(0xffffffffu, hbits, 1) << 16);
                            uint32_t wv[RPB / 2];
#pragma unroll
                            for (int i = 0; i < RPB / 2; ++i) wv[i] = __shfl_sync(0xffffffffu, word, 2 * i);
                            if (to_peer) {
                                uint8_t *dst = p.peer.out[lane] + (size_t)row0 * 2;
                                if constexpr (RPB % 8 == 0) {  // blocks start on 16-byte boundaries
#pragma unroll
                                    for (int i = 0; i < RPB / 8; ++i)
                                        reinterpret_cast<uint4 *>(dst)[i] = make_uint4(wv[4 * i], wv[4 * i + 1], wv[4 * i + 2], wv[4 * i + 3]);
                                } else {  // 14-row blocks start on 4-byte boundaries
#pragma unroll
                                    for (int i = 0; i < RPB / 2; ++i) reinterpret_cast<uint32_t *>(dst)[i] = wv[i];
                                }
                            }
                        } else {
                            uint32_t fv[RPB];
#pragma unroll
                            for (int i = 0; i < RPB; ++i) fv[i] = __shfl_sync(0xffffffffu, hbits, i);
                            if (to_peer) {
                                uint32_t *dst = reinterpret_cast<uint32_t *>(p.peer.out[lane] + (size_t)row0 * 4);
                                if constexpr (RPB % 4 == 0) {
#pragma unroll
                                    for (int i = 0; i < RPB / 4; ++i)
                                        reinterpret_cast<uint4 *>(dst)[i] = make_uint4(fv[4 * i], fv[4 * i + 1], fv[4 * i + 2], fv[4 * i + 3]);
                                } else {
#pragma unroll
                                    for (int i = 0; i < RPB / 2; ++i) reinterpret_cast<uint2 *>(dst)[i] = make_uint2(fv[2 * i], fv[2 * i + 1]);
                                }
                            }
                        }
                    } else if (live) {
                        // the bank's ragged last block: one store per row and peer
                        for (uint32_t r = 0; r < p.peer.world; ++r) {
                            if (r == p.peer.rank) continue;
                            if (p.out_bf16) {
                                reinterpret_cast<uint16_t *>(p.peer.out[r])[row] = (uint16_t)hbits;
                            } else {
                                reinterpret_cast<float *>(p.peer.out[r])[row] = v;
                            }
                        }
                    }
                }
            } else {
                // lane l: MMA row l / 2, batch columns 4 (l % 2) .. + 3
                const uint32_t r = lane >> 1, c0 = (lane & 1) * 4;
                float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int w = 0; w < kConsumers; ++w) {
                    const uint4 q = q4k::lds128(part + ((w * 16 + r) * 8 + c0) * 4);
                    v[0] += __uint_as_float(q.x), v[1] += __uint_as_float(q.y);
                    v[2] += __uint_as_float(q.z), v[3] += __uint_as_float(q.w);
                }
                const uint32_t row = row0 + 2 * (r & 7u) + (r >> 3);  // MMA row r holds local row 2 (r % 8) + r / 8
                if ((r & 7u) < (uint32_t)(ROWS / 2) && row < sg.rows) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t n = c0 + c;
                        if (n < p.m) {
                            float o = v[c];
                            const size_t idx = (size_t)n * sg.rows + row;
                            if (p.epi == q4k::EPI_ADD_RESID) o = o + sg.resid[idx];
                            if (p.out_bf16) {
                                static_cast<uint16_t *>(sg.out)[idx] = dev::f32_to_bf16_store(o);
                            } else {
                                static_cast<float *>(sg.out)[idx] = o;
                            }
                        }
                    }
                }
            }
            if constexpr (BATCH) {
                __syncwarp();
                if (lane == 0) mbar_arrive(empty(s));  // partial sums read: the stage may be refilled
            }
            if (++s == S) s = 0, ph ^= 1u;
        }
        if (peered && good) {
            uint32_t *mine = p.peer.flags[p.peer.rank];
            // Release in two steps, so that one system-scope fence is paid per launch and not one per block: each
            // block orders its peer stores before its ticket at DEVICE scope; the block that draws the last ticket
            // has then observed every block's ticket, and its one system-scope fence (cumulative over what it
            // observed) orders all those stores before the relaxed store of the completion flag.
            __threadfence();
            __syncwarp();
            uint32_t ticket = 0;
            if (lane == 0) ticket = atomicAdd(mine + 17, 1u);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            __syncwarp();  // lane 0's observation of the tickets, ordered before the other lanes' fences and stores
            if (ticket == gridDim.x - 1) {
                __threadfence_system();
                if ((uint32_t)lane < p.peer.world && (uint32_t)lane != p.peer.rank)
                    st_relaxed_sys(p.peer.flags[lane] + 8 + p.peer.rank, seq);
                const bool done = p.peer.defer != 0 ||
                                  peer_wait(mine, p.peer.rank, p.peer.world, p.peer.wait_clocks, p.status, 8, seq, 4);
                if (done && lane == 0) mine[17] = 0, mine[16] = seq;
            }
        }
    } else {
        // ------------------------------------------------ consumers ---
        const uint32_t g = lane >> 2, t = lane & 3;
        const uint32_t KW = K / NWIN;                             // columns of one window
        const uint32_t k0 = (uint32_t)warp * (KW / kConsumers);  // first column of this warp's slice within a window
        const uint32_t G = 1u << p.group_shift;
        // x is written by the preceding kernel in a decode chain: wait for it.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (p.xwait_world > 1) {
            // x is a gathered vector whose exchange did not wait for the peers: their slices are here once their
            // completion flags have reached this rank's call counter (final: the exchanging kernel has finished)
            // One warp polls and pays the system-scope acquire (hidden behind the weight prefetch; taken by every
            // consumer warp of every block at once it cost the launch 14 us); the block-scope barrier hands its
            // effect to the other consumer warps.
            if (warp == 0) {
                const uint32_t seq = *(volatile const uint32_t *)(p.xwait.flags + 16);
                if (!peer_wait(p.xwait.flags, p.xwait.rank, p.xwait.world, p.xwait.wait_clocks, p.status, 8, seq, 5))
                    *abortp = 1;  // the other roles leave their loops; nothing is computed from an incomplete x
                else
                    __threadfence_system();
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");
            if (*abortp) return;
        }
        // B fragments of the slice: word (jj, u) of this lane covers columns
        // k0 + jj G + t G / 4 + 8 u .. + 7, in the order 0,4,1,5,2,6,3,7 that the
        // nibble-pair extraction below produces.
        uint32_t xb[SW][4];
        float xs[NGS];  // group sums of the activations: column g (BATCH) or the vector (M = 1)
        // Q4: the nibbles go to the MMA as the bf16 bit patterns 0..15 and 16 x (0..15), i.e. q * 2^-133 (the
        // subnormal range and the first binade of bf16 are one linear scale), so the activations carry the
        // rest: times 2^e (e puts the slice's largest magnitude of this row of x near 2^100, so that every
        // product is a normal f32), the partners of the odd nibbles divided by 16 as well. Both are changes
        // of the exponent field only, hence exact; `cw` = 2^(133 - e) undoes them in the fold.
        float cw = 0.0f;
        float cwv[NWIN];  // per window (M = 1)
        // this lane's B fragments and group sums of window `win`, from the warp's staged copy
        auto load_x = [&](int win) {
            const uint32_t xst = xstage + win * kXStageBytes;
#pragma unroll
            for (int jj = 0; jj < NGS; ++jj) {
#pragma unroll
                for (int u = 0; u < WPG; ++u) {
                    const uint4 f = q4k::lds128(xst + (jj * 4 * WPG + t * WPG + u) * 16);
                    xb[jj * WPG + u][0] = f.x, xb[jj * WPG + u][1] = f.y, xb[jj * WPG + u][2] = f.z, xb[jj * WPG + u][3] = f.w;
                }
                xs[jj] = __uint_as_float(lds32(xst + 512 + jj * 4));
            }
        };
        {
            const uint32_t n = BATCH ? min(g, p.m - 1) : 0u;
            const uint16_t *xrow = p.x + (size_t)n * p.x_pitch;
            int e = 0;
            if constexpr (BATCH || Q8) {
                uint32_t amax = 0;
#pragma unroll
                for (int jj = 0; jj < NGS; ++jj) {
#pragma unroll
                    for (int u = 0; u < WPG; ++u) {
                        const uint32_t k = k0 + jj * G + t * (G / 4) + 8 * u;
                        if constexpr (Q8) {
                            const uint2 r = __ldg(reinterpret_cast<const uint2 *>(xrow + k / 2));
                            amax = max(amax, max(max(r.x & 0x7fffu, (r.x >> 16) & 0x7fffu), max(r.y & 0x7fffu, (r.y >> 16) & 0x7fffu)));
                        } else {
                            const uint4 r = __ldg(reinterpret_cast<const uint4 *>(xrow + k));
                            amax = max(amax, max(max(r.x & 0x7fffu, (r.x >> 16) & 0x7fffu), max(r.y & 0x7fffu, (r.y >> 16) & 0x7fffu)));
                            amax = max(amax, max(max(r.z & 0x7fffu, (r.z >> 16) & 0x7fffu), max(r.w & 0x7fffu, (r.w >> 16) & 0x7fffu)));
                        }
                    }
                }
                amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                if ((amax >> 7) != 0) {
                    const int maxexp = (int)(amax >> 7) - 127;
                    e = min(126, max(100, maxexp + 6)) - maxexp;
                    cw = __uint_as_float((uint32_t)(127 + 133 - e) << 23);
                }
            }
            // bf16 bits times 2^ee; zeros, subnormals and whatever would leave the normal range become 0
            auto scaled = [](uint32_t b, int ee) -> uint32_t {
                const int ex = (int)((b >> 7) & 0xffu), nx = ex + ee;
                return (ex == 0 || nx < 1 || nx > 254) ? 0u : ((b & 0x807fu) | ((uint32_t)nx << 7));
            };
            auto pair = [&](uint32_t lo, uint32_t hi, int ee) { return scaled(lo & 0xffffu, ee) | (scaled(hi & 0xffffu, ee) << 16); };
            if constexpr (!BATCH && !Q8) {
                constexpr uint32_t NW = 4 * SW;  // 8-column words of the slice: lane L < NW handles word L
                // Every window's load first, then the processing: one L2 round trip on the launch's start-up path
                // instead of one per window (the loads are volatile: the compiler would not move them).
                uint4 rw[NWIN];
#pragma unroll
                for (int win = 0; win < NWIN; ++win) {
                    rw[win] = make_uint4(0u, 0u, 0u, 0u);
                    // a coherent load: x may be a gather buffer that a peer GPU filled while this kernel was waiting
                    if ((uint32_t)lane < NW) {
                        asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(rw[win].x), "=r"(rw[win].y), "=r"(rw[win].z), "=r"(rw[win].w)
                                     : "l"(xrow + win * KW + k0 + 8 * lane)
                                     : "memory");
                    }
                }
#pragma unroll
                for (int win = 0; win < NWIN; ++win) {
                    const uint32_t xst = xstage + win * kXStageBytes;
                    const uint4 r = rw[win];
                    uint32_t amax = max(max(r.x & 0x7fffu, (r.x >> 16) & 0x7fffu), max(r.y & 0x7fffu, (r.y >> 16) & 0x7fffu));
                    amax = max(amax, max(max(r.z & 0x7fffu, (r.z >> 16) & 0x7fffu), max(r.w & 0x7fffu, (r.w >> 16) & 0x7fffu)));
                    amax = __reduce_max_sync(0xffffffffu, amax);  // one instruction: this chain is the launch's start-up path
                    e = 0, cw = 0.0f;
                    if ((amax >> 7) != 0) {
                        const int maxexp = (int)(amax >> 7) - 127;
                        e = min(126, max(100, maxexp + 6)) - maxexp;
                        cw = __uint_as_float((uint32_t)(127 + 133 - e) << 23);
                    }
                    cwv[win] = cw;
                    if ((uint32_t)lane < NW) {
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(xst + lane * 16), "r"(pair(r.x, r.z, e)),
                                     "r"(pair(r.x >> 16, r.z >> 16, e - 4)), "r"(pair(r.y, r.w, e)), "r"(pair(r.y >> 16, r.w >> 16, e - 4))
                                     : "memory");
                    }
                    float part = (dev::bf16_lo(r.x) + dev::bf16_hi(r.x)) + (dev::bf16_lo(r.y) + dev::bf16_hi(r.y));
                    part += (dev::bf16_lo(r.z) + dev::bf16_hi(r.z)) + (dev::bf16_lo(r.w) + dev::bf16_hi(r.w));
#pragma unroll
                    for (int o = 1; o < 4 * WPG && o < 32; o <<= 1) part += __shfl_xor_sync(0xffffffffu, part, o);  // a group: 4 WPG lanes
                    const float gsum = __shfl_sync(0xffffffffu, part, (lane * 4 * WPG) & 31);
                    if (lane < NGS) asm volatile("st.shared.f32 [%0], %1;" ::"r"(xst + 512 + lane * 4), "f"(gsum) : "memory");
                }
                __syncwarp();
                if constexpr (NWIN == 1) load_x(0);
            } else
#pragma unroll
            for (int jj = 0; jj < NGS; ++jj) {
                float part = 0.0f;
#pragma unroll
                for (int u = 0; u < WPG; ++u) {
                    const uint32_t k = k0 + jj * G + t * (G / 4) + 8 * u;
                    if constexpr (Q8) {
                        // the word holds 4 codes; a code 0..255 read as a bf16 bit pattern is c * 2^-133 exactly (the
                        // subnormals and the first binade form one linear scale), so (w & 0x00ff00ff) is an A register
                        // of codes 0, 2 and ((w >> 8) & 0x00ff00ff) one of codes 1, 3: no magic constant, no offset
                        const uint2 r = __ldg(reinterpret_cast<const uint2 *>(xrow + k / 2));
                        xb[jj * WPG + u][0] = pair(r.x, r.y, e);              // x0, x2
                        xb[jj * WPG + u][1] = pair(r.x >> 16, r.y >> 16, e);  // x1, x3
                        part += (dev::bf16_lo(r.x) + dev::bf16_hi(r.x)) + (dev::bf16_lo(r.y) + dev::bf16_hi(r.y));
                    } else {
                        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(xrow + k));
                        xb[jj * WPG + u][0] = pair(r.x, r.z, e);                  // x0, x4
                        xb[jj * WPG + u][1] = pair(r.x >> 16, r.z >> 16, e - 4);  // (x1, x5) / 16
                        xb[jj * WPG + u][2] = pair(r.y, r.w, e);                  // x2, x6
                        xb[jj * WPG + u][3] = pair(r.y >> 16, r.w >> 16, e - 4);  // (x3, x7) / 16
                        part += (dev::bf16_lo(r.x) + dev::bf16_hi(r.x)) + (dev::bf16_lo(r.y) + dev::bf16_hi(r.y));
                        part += (dev::bf16_lo(r.z) + dev::bf16_hi(r.z)) + (dev::bf16_lo(r.w) + dev::bf16_hi(r.w));
                    }
                }
                part += __shfl_xor_sync(0xffffffffu, part, 1);
                part += __shfl_xor_sync(0xffffffffu, part, 2);
                xs[jj] = part;  // the same in the four lanes of a quad
            }
        }
        // BATCH: this lane's outputs are batch columns 2 t and 2 t + 1; their group sums live in quads 2 t and 2 t + 1.
        float xs0[BATCH ? NGS : 1], xs1[BATCH ? NGS : 1];
        float cw0 = cw, cw1 = cw;  // the multipliers of this lane's two output columns
        if constexpr (BATCH) {
            cw0 = __shfl_sync(0xffffffffu, cw, (2 * t) * 4);
            cw1 = __shfl_sync(0xffffffffu, cw, (2 * t + 1) * 4);
#pragma unroll
            for (int jj = 0; jj < NGS; ++jj) {
                xs0[jj] = __shfl_sync(0xffffffffu, xs[jj], (2 * t) * 4);
                xs1[jj] = __shfl_sync(0xffffffffu, xs[jj], (2 * t + 1) * 4);
            }
        }
        if (lane == 0) mbar_arrive(xbar);  // this warp holds its x fragments: the producer may fill the rest of the ring
        const uint32_t w_off = (k0 >> 1) + t * (G / 8);  // byte offset of the lane's first word within a row
        const uint32_t sb_off = (k0 >> p.group_shift) * 4;

        // lane groups beyond the stage's row pairs (ROWS < 16) read the last pair again: their MMA rows are never stored
        const uint32_t gp = min(g, (uint32_t)(ROWS / 2 - 1));
        const uint32_t row_base = pair_off(gp) + w_off, sb_base = sb_pair_off(gp) + sb_off;  // within a stage
        uint32_t s = 0, ph = 0;
        for (uint32_t j = 0; j < n_local; ++j) {
            if (!mbar_wait(full(s), ph, abortp, 32)) {  // sleeping between polls leaves issue slots to the producer
                if (lane == 0) fail(2, j);
                break;
            }
            const uint32_t st = ring + s * stage_bytes;
            float vlo = 0.0f, vhi = 0.0f;  // M = 1: this lane's share of MMA rows g and g + 8, over all windows
            float acc[4][4] = {};
#pragma unroll
            for (int win = 0; win < NWIN; ++win) {
            if constexpr (NWIN > 1) load_x(win), cw = cwv[win];
            const uint32_t row_lo = st + row_base + win * (KW >> 1), row_hi = row_lo + row_bytes;
            const uint32_t sb_lo = st + sb_base + win * ((KW >> p.group_shift) * 4);
            const uint32_t sb_hi = sb_lo + sb_row_bytes;
            float dlo[NGS], dhi[NGS];        // M = 1: dot of MMA rows g and g + 8 per group
            // BATCH: rows g, g + 8 x columns 2 t, 2 t + 1, one accumulator per group class jj % 4 so that
            // the sum is formed in the same order as in the M = 1 path (where lane t of a quad takes
            // the groups t, t + 4, ... and the quad is then added up by a butterfly)
            // All words of the slice first (the rows were copied long ago: these loads do not wait),
            // then the MMAs interleaved over the groups: consecutive MMAs belong to different
            // accumulator chains, so none waits for its predecessor. Within a chain the order is
            // word by word, first half before second, whatever the interleaving.
            uint32_t wl[SW], wh[SW];
#pragma unroll
            for (int jj = 0; jj < NGS; ++jj) {
                if constexpr (WPG >= 2) {
#pragma unroll
                    for (int u2 = 0; u2 < WPG; u2 += 2) {
                        const uint2 a = lds64(row_lo + jj * (G / 2) + 4 * u2), b = lds64(row_hi + jj * (G / 2) + 4 * u2);
                        wl[jj * WPG + u2] = a.x, wl[jj * WPG + u2 + 1] = a.y;
                        wh[jj * WPG + u2] = b.x, wh[jj * WPG + u2 + 1] = b.y;
                    }
                } else {
                    wl[jj] = lds32(row_lo + jj * (G / 2)), wh[jj] = lds32(row_hi + jj * (G / 2));
                }
            }
            float d[NGS][4] = {};
#pragma unroll
            for (int u = 0; u < WPG; ++u) {
#pragma unroll
                for (int jj = 0; jj < NGS; ++jj) {
                    const uint32_t a = wl[jj * WPG + u], b = wh[jj * WPG + u];
                    if constexpr (Q8) {
                        mma_bf16(d[jj], a & 0x00ff00ffu, b & 0x00ff00ffu, (a >> 8) & 0x00ff00ffu, (b >> 8) & 0x00ff00ffu,
                                 xb[jj * WPG + u][0], xb[jj * WPG + u][1]);  // codes 0,2 | 1,3
                    } else {
                        // nibble pairs (0, 4) and 16 x (1, 5) in place: five ALU instructions per word instead of
                        // seven (these share the busiest pipe of the kernel), and nothing to subtract afterwards
                        mma_bf16(d[jj], a & 0x000f000fu, b & 0x000f000fu, a & 0x00f000f0u, b & 0x00f000f0u, xb[jj * WPG + u][0],
                                 xb[jj * WPG + u][1]);
                    }
                }
#pragma unroll
                for (int jj = 0; jj < NGS; ++jj) {
                    const uint32_t a = wl[jj * WPG + u], b = wh[jj * WPG + u];
                    if constexpr (!Q8) {
                        const uint32_t as = a >> 8, bs = b >> 8;
                        mma_bf16(d[jj], as & 0x000f000fu, bs & 0x000f000fu, as & 0x00f000f0u, bs & 0x00f000f0u, xb[jj * WPG + u][2],
                                 xb[jj * WPG + u][3]);
                    }
                }
            }
#pragma unroll
            for (int jj = 0; jj < NGS; ++jj) {
                if constexpr (BATCH) {
                    const uint32_t pl = lds32(sb_lo + jj * 4), ph2 = lds32(sb_hi + jj * 4);
                    const float sl = dev::bf16_lo(pl), bl = dev::bf16_hi(pl), sh = dev::bf16_lo(ph2), bh = dev::bf16_hi(ph2);
                    const int cls = jj & 3;  // a constant once the loop is unrolled
                    acc[0][cls] = fmaf(sl, d[jj][0] * cw0, fmaf(bl, xs0[jj], acc[0][cls]));
                    acc[1][cls] = fmaf(sl, d[jj][1] * cw1, fmaf(bl, xs1[jj], acc[1][cls]));
                    acc[2][cls] = fmaf(sh, d[jj][2] * cw0, fmaf(bh, xs0[jj], acc[2][cls]));
                    acc[3][cls] = fmaf(sh, d[jj][3] * cw1, fmaf(bh, xs1[jj], acc[3][cls]));
                } else {
                    dlo[jj] = d[jj][0], dhi[jj] = d[jj][2];  // every column holds the same vector: d[1] == d[0]
                }
            }
            if constexpr (!BATCH) {
                // The four lanes of a quad hold the same dots: lane t folds the affine of groups t, t + 4, ...
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    float dl = 0.0f, dh = 0.0f, xg = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (4 * q + i < NGS && t == (uint32_t)i) dl = dlo[4 * q + i], dh = dhi[4 * q + i], xg = xs[4 * q + i];
                    const uint32_t jj = 4 * q + t;
                    if (jj < (uint32_t)NGS) {
                        const uint32_t pl = lds32(sb_lo + jj * 4), ph2 = lds32(sb_hi + jj * 4);
                        vlo = fmaf(dev::bf16_lo(pl), dl * cw, fmaf(dev::bf16_hi(pl), xg, vlo));
                        vhi = fmaf(dev::bf16_lo(ph2), dh * cw, fmaf(dev::bf16_hi(ph2), xg, vhi));
                    }
                }
            }
            }  // windows
            const uint32_t part = st + off_part;
            if constexpr (BATCH) {
                float o[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) o[c] = (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]);
                asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(part + ((warp * 16 + g) * 8 + 2 * t) * 4), "f"(o[0]),
                             "f"(o[1])
                             : "memory");
                asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(part + ((warp * 16 + g + 8) * 8 + 2 * t) * 4),
                             "f"(o[2]), "f"(o[3])
                             : "memory");
            } else {
                vlo += __shfl_xor_sync(0xffffffffu, vlo, 1), vhi += __shfl_xor_sync(0xffffffffu, vhi, 1);
                vlo += __shfl_xor_sync(0xffffffffu, vlo, 2), vhi += __shfl_xor_sync(0xffffffffu, vhi, 2);
                if (t == 0) {
                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(part + (warp * 16 + g) * 4), "f"(vlo) : "memory");
                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(part + (warp * 16 + g + 8) * 4), "f"(vhi) : "memory");
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(done(s));  // release: the partial sums are visible to the reducer
            if (++s == S) s = 0, ph ^= 1u;
        }
    }
}

}  // namespace q4m
}  // namespace tessl
