// Pieces shared by the prefill GEMM kernels (single-CTA and CTA-pair): the launch
// parameters, the PTX wrappers for TMA, tcgen05 and f16x2 arithmetic, and the
// nibble -> f16 expansion of one packed weight row.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "q4_gemv_tma.cuh"
#include "runtime.h"

namespace tessl {
namespace pf {

using q4k::and_or;
using q4k::lds128;
using q4k::mbar_arrive;
using q4k::mbar_expect_tx;
using q4k::mbar_init;
using q4k::mbar_try;
using q4k::mbar_wait;
using q4k::smem_u32;

constexpr int BM = 128;  // rows of X per tile = MMA M
constexpr int BK = 64;   // K block: 128 bytes of f16 = one swizzle row
constexpr uint32_t kTmemCols = 512;

struct GemmParams {
    const uint32_t *sb;   // bf16 (scale, bias) pairs [N, K / G]
    const float *row_scale;  // [M] power-of-two scale removed from each X row
    void *y;
    uint32_t M, N, K;
    uint32_t gshift;       // log2 G
    uint32_t gpr;          // K / G
    uint32_t nkb_main;     // ceil(K / 64)
    uint32_t nkb_extra;    // ceil(4 * gpr / 64)
    uint32_t tiles_m, tiles_n;
    int out_bf16;
    uint32_t *status;
};


// ---------------------------------------------------------------- PTX wrappers ---

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
/// D[tmem] (+)= A[smem] . B[smem]^T for one K = 16 slice.
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
/// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 B
/// apart, 8-row groups 1024 B apart, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t pack_h2(__half lo, __half hi)
{
    return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

// ------------------------------------------------- weight expansion, stores ---

/// NW packed words (8 nibbles each) of one weight row -> 8 NW f16 values
/// s * (q - 8), written as 16-byte chunks c0 .. c0 + NW - 1 of the 128-byte row at
/// `brow` with the 128B swizzle (`swz` = (row & 7) << 4). `s` is the group scale
/// as an f16 pair. Each chunk holds the eight weights of one packed word in the
/// order 0,4,1,5,2,6,3,7.
template <int NW>
__device__ __forceinline__ void expand_q4_words(const uint32_t (&words)[NW], uint32_t s, uint32_t brow, uint32_t swz,
                                                uint32_t c0)
{
#pragma unroll
    for (int c = 0; c < NW; ++c) {
        const uint32_t w = words[c], w8 = w >> 8;
        // (1024 + q) and (1024 + 16 q) as f16 pairs, then q - 8 exactly, then * s exactly
        const uint32_t t0 = and_or(w, 0x000f000fu, 0x64006400u);
        const uint32_t t1 = and_or(w, 0x00f000f0u, 0x64006400u);
        const uint32_t t2 = and_or(w8, 0x000f000fu, 0x64006400u);
        const uint32_t t3 = and_or(w8, 0x00f000f0u, 0x64006400u);
        const uint32_t ox = h2_mul(h2_sub(t0, 0x64086408u), s);                // 1024 + q - 1032
        const uint32_t oy = h2_mul(h2_fma(t1, 0x2c002c00u, 0xd480d480u), s);  // (1024 + 16 q) / 16 - 72
        const uint32_t oz = h2_mul(h2_sub(t2, 0x64086408u), s);
        const uint32_t ow = h2_mul(h2_fma(t3, 0x2c002c00u, 0xd480d480u), s);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(brow + (((c0 + (uint32_t)c) << 4) ^ swz)), "r"(ox),
                     "r"(oy), "r"(oz), "r"(ow)
                     : "memory");
    }
}

/// The f16 pair (scale, scale) of a bf16 (scale, bias) word.
__device__ __forceinline__ uint32_t scale_h2(uint32_t pair)
{
    const __half sh = __float2half_rn(dev::bf16_lo(pair));
    return pack_h2(sh, sh);
}

/// Chunks c0 .. c0 + NC - 1 of extra K block `e` of one weight row: per group
/// (c1, c1, c1, c2) with c1 + c2 the two-piece f16 split of b + 8 s, two groups
/// per chunk; groups past `gpr` are zero.
template <int NC>
__device__ __forceinline__ void expand_extra_chunks(const uint32_t *sbrow, uint32_t e, uint32_t gpr, uint32_t brow,
                                                    uint32_t swz, uint32_t c0)
{
#pragma unroll
    for (int cc = 0; cc < NC; ++cc) {
        const uint32_t c = c0 + (uint32_t)cc;
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t g = e * 16 + 2 * c + j;
            uint32_t lo = 0, hi = 0;
            if (g < gpr) {
                const uint32_t pair = __ldg(sbrow + g);
                const float bp = fmaf(8.0f, dev::bf16_lo(pair), dev::bf16_hi(pair));
                const __half c1 = __float2half_rn(bp);
                const __half c2 = __float2half_rn(bp - __half2float(c1));
                lo = pack_h2(c1, c1), hi = pack_h2(c1, c2);
            }
            o[2 * j] = lo, o[2 * j + 1] = hi;
        }
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(brow + ((c << 4) ^ swz)), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                     "r"(o[3])
                     : "memory");
    }
}

/// 32 consecutive accumulator columns of output row `m`, columns n .. n + 31:
/// undo the row scale and store as f32 or bf16.
__device__ __forceinline__ void store_row32(const GemmParams &p, const uint32_t (&r)[32], uint32_t m, uint32_t n, float rs)
{
    if (m >= p.M || n >= p.N) return;
    if (p.out_bf16) {
        uint16_t *dst = static_cast<uint16_t *>(p.y) + (size_t)m * p.N + n;
        if ((p.N & 7u) == 0 && n + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 o;
                uint32_t *ow = &o.x;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    ow[k] = (uint32_t)dev::f32_to_bf16_store(__uint_as_float(r[8 * j + 2 * k]) * rs) |
                            ((uint32_t)dev::f32_to_bf16_store(__uint_as_float(r[8 * j + 2 * k + 1]) * rs) << 16);
                reinterpret_cast<uint4 *>(dst)[j] = o;
            }
        } else {
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j)  // unrolled: the accumulator values stay in registers
                if (n + j < p.N) dst[j] = dev::f32_to_bf16_store(__uint_as_float(r[j]) * rs);
        }
    } else {
        float *dst = static_cast<float *>(p.y) + (size_t)m * p.N + n;
        if ((p.N & 3u) == 0 && n + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                reinterpret_cast<float4 *>(dst)[j] =
                    make_float4(__uint_as_float(r[4 * j]) * rs, __uint_as_float(r[4 * j + 1]) * rs,
                                __uint_as_float(r[4 * j + 2]) * rs, __uint_as_float(r[4 * j + 3]) * rs);
        } else {
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j)
                if (n + j < p.N) dst[j] = __uint_as_float(r[j]) * rs;
        }
    }
}

/// The same 32 x 32 block of outputs as 32 calls of store_row32 (lane = row
/// m_base + lane, columns n .. n + 31), but written with full 128-byte lines: the
/// warp transposes the block through `stage` (4 KiB of shared memory of its own,
/// 16-byte chunks XOR-swizzled so both phases are bank-conflict free) and each
/// store instruction then covers whole rows segments instead of 32 scattered
/// 16-byte pieces. Falls back to the per-row path for ragged widths.
__device__ __forceinline__ void store_block32_coalesced(const GemmParams &p, const uint32_t (&r)[32], uint32_t stage,
                                                        uint32_t lane, uint32_t m_base, uint32_t n, float rs)
{
    if (n >= p.N) return;
    if (!p.out_bf16 && (p.N & 3u) == 0 && n + 32 <= p.N) {
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            const uint32_t a = stage + lane * 128 + ((j ^ (lane & 7u)) << 4);
            asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(a), "f"(__uint_as_float(r[4 * j]) * rs),
                         "f"(__uint_as_float(r[4 * j + 1]) * rs), "f"(__uint_as_float(r[4 * j + 2]) * rs),
                         "f"(__uint_as_float(r[4 * j + 3]) * rs)
                         : "memory");
        }
        __syncwarp();
        const uint32_t cj = lane & 7u, rsub = lane >> 3;
        float *y = static_cast<float *>(p.y);
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t row = 4 * i + rsub;
            const uint4 v = lds128(stage + row * 128 + ((cj ^ (row & 7u)) << 4));
            if (m_base + row < p.M) *reinterpret_cast<uint4 *>(y + (size_t)(m_base + row) * p.N + n + 4 * cj) = v;
        }
        __syncwarp();
    } else if (p.out_bf16 && (p.N & 7u) == 0 && n + 32 <= p.N) {
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                o[k] = (uint32_t)dev::f32_to_bf16_store(__uint_as_float(r[8 * j + 2 * k]) * rs) |
                       ((uint32_t)dev::f32_to_bf16_store(__uint_as_float(r[8 * j + 2 * k + 1]) * rs) << 16);
            const uint32_t a = stage + lane * 64 + ((j ^ ((lane >> 1) & 3u)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                         : "memory");
        }
        __syncwarp();
        const uint32_t cj = lane & 3u, rsub = lane >> 2;
        uint16_t *y = static_cast<uint16_t *>(p.y);
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t row = 8 * i + rsub;
            const uint4 v = lds128(stage + row * 64 + ((cj ^ ((row >> 1) & 3u)) << 4));
            if (m_base + row < p.M) *reinterpret_cast<uint4 *>(y + (size_t)(m_base + row) * p.N + n + 8 * cj) = v;
        }
        __syncwarp();
    } else {
        store_row32(p, r, m_base + lane, n, rs);
    }
}

// ------------------------------------------------------ CTA-pair (cluster) PTX ---

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
/// The shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
/// Arrive on an mbarrier given by its shared::cluster address (this CTA's or the peer's).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
/// TMA tile load issued by one CTA of a pair into its own shared memory; the
/// completion bytes are signalled on `bar`, a shared::cluster address that may be
/// the peer's barrier. Each CTA fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
        "[%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
/// D[tmem of both CTAs] (+)= A . B^T, M = 256 over the pair (128 rows per CTA), each CTA supplying half of B's rows.
__device__ __forceinline__ void tcgen05_mma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
/// Arrive on a barrier of the issuing (leader) CTA only, once all pair MMAs issued so far have completed.
__device__ __forceinline__ void tcgen05_commit_pair_local(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
/// Arrive, once all MMAs issued so far have completed, on the barrier at this
/// shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(mask)
        : "memory");
}

/// Position in a ring of S stages with the parity of its current round; advancing
/// wraps without a division (the role loops run once per K block).
template <int S>
struct RingPos {
    uint32_t stage = 0, phase = 0;
    __device__ __forceinline__ void advance(uint32_t n = 1)  // n <= S
    {
        stage += n;
        if (stage >= (uint32_t)S) stage -= (uint32_t)S, phase ^= 1u;
    }
    __device__ __forceinline__ void set(uint32_t index) { stage = index % (uint32_t)S, phase = (index / (uint32_t)S) & 1u; }
};

/// Low word of the shared-memory matrix descriptor of a K-major, 128B-swizzled
/// tile at `smem_addr`; the high word is kUmmaDescHi for every such tile.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3ffffu) >> 4) | (1u << 16); }
constexpr uint32_t kUmmaDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);

/// Pair MMA with the descriptors given by their low words.
__device__ __forceinline__ void tcgen05_mma_f16_pair_lo(uint32_t tmem_d, uint32_t adesc_lo, uint32_t bdesc_lo, uint32_t idesc,
                                                        uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(adesc_lo), "r"(bdesc_lo), "r"(idesc), "r"(accumulate), "r"(kUmmaDescHi)
        : "memory");
}

// Warp-wide forms for an issuing warp that stays converged: all 32 lanes execute
// the surrounding loop (so stage numbers and descriptors are warp-uniform values)
// and one elected lane, always the same one, issues the instruction.
__device__ __forceinline__ void tcgen05_mma_f16_pair_elect(uint32_t tmem_d, uint32_t adesc_lo, uint32_t bdesc_lo,
                                                           uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(adesc_lo), "r"(bdesc_lo), "r"(idesc), "r"(accumulate), "r"(kUmmaDescHi)
        : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair_elect(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile(
        "{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}" ::"r"(
            bar),
        "h"(mask)
        : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair_local_elect(uint32_t bar)
{
    asm volatile(
        "{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar)
        : "memory");
}

}  // namespace pf
}  // namespace tessl
