// MLX Q4 prefill GEMM, CTA-pair form: two CTAs on neighbouring SMs (a cluster of
// two) compute one 256 x BN output tile with tcgen05.mma.cta_group::2. Same math
// and operand layouts as the single-CTA kernel in prefill_gemm.cu; what changes
// is who holds what:
//
//   * each CTA loads its own 128 rows of the f16 activations (A) by TMA and
//     dequantizes only its own BN/2 weight rows (half of B) into shared memory;
//     the pair's MMA reads A from both CTAs and both halves of B, so per output
//     element the shared-memory traffic, the L2 traffic for weights and the
//     dequant arithmetic are half of the single-CTA kernel's;
//   * the even CTA (rank 0, the leader) issues every MMA. The barriers it waits
//     on live in its shared memory: A tiles of both CTAs complete their bytes
//     there, and the peer's dequant and epilogue warps arrive there through the
//     cluster address. The barriers the other roles wait on (stage free,
//     accumulator ready) exist in both CTAs at the same offset and are signalled
//     together by tcgen05.commit with a two-CTA mask;
//   * each CTA's TMEM holds its 128 rows x BN columns of the accumulator, twice
//     (double buffered), so the epilogue of one tile overlaps the next main loop.
//
// Roles per CTA: warp 0 TMA producer of the X tiles, warp 1 TMEM allocation (+ MMA
// issue in the leader), warp 2 TMA producer of the packed weights (its own, deeper
// ring: the dequant warps need a block's nibbles long before the MMA needs its X
// tile), warp 3 idle, warps 4-7 epilogue (each transposes its 32 x 32 blocks through
// 4 KiB of shared memory so that the stores are whole lines), then two groups of BN/32 dequant warps
// that take alternate K blocks, two threads per weight row (32 weights each).
// Every wait is bounded; on a timeout the status word is set and all roles fall
// through to the closing cluster barrier.
#pragma once
#include "prefill_common.cuh"

namespace tessl {
namespace pf {

template <int BN>
struct PairCfg {
    static constexpr int HB = BN / 2;                 // weight rows this CTA expands
    static constexpr int SA = 6;                      // stages of the (X tile, dequantized-W tile) ring
    static constexpr int SB = SA;                     // one ring: a K block's two operands are freed together
    static constexpr int SQ = BN == 256 ? 4 : 8;      // packed-W stages
    static constexpr int NDW = HB / 16;               // dequant warps per group (two threads per weight row)
    static constexpr int NG = 2;                      // dequant groups; group g expands K blocks g, g + 2, ...
    static constexpr int FIRST_DW = 8;                // first dequant warp
    static constexpr int THREADS = (FIRST_DW + NG * NDW) * 32;
    // Sleep between mbarrier polls (ns) of the roles that run ahead of the MMA issuer.
    static constexpr uint32_t POLL_PRODUCER = 100, POLL_DEQUANT = 40, POLL_EPILOGUE = 400;
    static constexpr uint32_t A_BYTES = BM * BK * 2;  // 16 KiB
    static constexpr uint32_t Q_BYTES = HB * 32;
    static constexpr uint32_t B_BYTES = HB * BK * 2;
    static constexpr uint32_t OFF_A = 0;
    static constexpr uint32_t OFF_B = OFF_A + SA * A_BYTES;
    static constexpr uint32_t OFF_Q = OFF_B + SB * B_BYTES;
    static constexpr uint32_t OFF_STAGE = OFF_Q + SQ * Q_BYTES;  // 4 KiB per epilogue warp, to transpose its stores
    static constexpr uint32_t OFF_BAR = OFF_STAGE + 4 * 4096;
    static constexpr int NBARS = 2 * SA + 2 * SQ + 4 + 1;
    static constexpr uint32_t SMEM = OFF_BAR + NBARS * 8 + 1024;  // + slack to align the base to 1 KiB
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<BN>::THREADS, 1)
    q4_prefill_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                                const GemmParams p)
{
    using C = PairCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const uint32_t bar0 = base + C::OFF_BAR;
    // Offsets of the barriers; the same in both CTAs.
    //   full[s]    the leader's: stage s holds both CTAs' X tiles (TMA bytes) and both halves of B
    //              (one arrival per dequant warp of either CTA, one from the leader's producer)
    //   empty[s]   both CTAs': the MMAs that read stage s have completed (one commit frees A and B)
    //   q_full / q_empty   CTA-local ring of packed weight tiles
    //   acc_full[b] both CTAs'; acc_empty[b] the leader's (4 epilogue warps of either CTA)
    auto full = [&](uint32_t s) { return bar0 + 8 * s; };
    auto empty = [&](uint32_t s) { return bar0 + 8 * (C::SA + s); };
    auto q_full = [&](uint32_t s) { return bar0 + 8 * (2 * C::SA + s); };
    auto q_empty = [&](uint32_t s) { return bar0 + 8 * (2 * C::SA + C::SQ + s); };
    auto acc_full = [&](uint32_t b) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + b); };
    auto acc_empty = [&](uint32_t b) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + 2 + b); };
    const uint32_t done_bar = bar0 + 8 * (2 * C::SA + 2 * C::SQ + 4);
    // The leader's barrier block as seen from this CTA (its own block when this CTA leads).
    const uint32_t lead_delta = map_to_cta(bar0, 0) - bar0;

    const uint32_t nkb = p.nkb_main + p.nkb_extra;
    const uint32_t ntiles = p.tiles_m * p.tiles_n;  // pair tiles: tiles_m counts 256-row blocks
    const uint32_t cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (uint32_t s = 0; s < C::SA; ++s) mbar_init(full(s), 1 + 2 * C::NDW), mbar_init(empty(s), 1);
        for (uint32_t s = 0; s < C::SQ; ++s) mbar_init(q_full(s), 1), mbar_init(q_empty(s), C::NDW);
        for (uint32_t b = 0; b < 2; ++b) mbar_init(acc_full(b), 1), mbar_init(acc_empty(b), 8);
        mbar_init(done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anything can signal them
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;
    auto fail = [&](uint32_t role, uint32_t where) {
        *abortp = 1;
        *(volatile uint32_t *)p.status = (role << 24) | (rank << 23) | (where & 0x7fffffu);
    };

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: X tiles ---
        if (lane == 0) {
            RingPos<C::SA> ring;
            bool ok_ = true;
            for (uint32_t t = cluster_id; t < ntiles && ok_; t += nclusters) {
                const int m0 = (int)((t % p.tiles_m) * 2 + rank) * BM;
                for (uint32_t kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(empty(ring.stage), ring.phase ^ 1u, abortp, C::POLL_PRODUCER)) {
                        fail(1, kb);
                        ok_ = false;
                        break;
                    }
                    // The leader expects both CTAs' tiles on its barrier; either CTA's bytes may land first.
                    if (rank == 0) mbar_expect_tx(full(ring.stage), 2 * C::A_BYTES);
                    tma_load_2d_pair(base + C::OFF_A + ring.stage * C::A_BYTES, &map_a, (int)(kb * BK), m0,
                                     full(ring.stage) + lead_delta);
                    ring.advance();
                }
            }
            // These copies are covered by the leader's wait for its last MMA, which has read them all.
        }
    } else if (warp == 2) {
        // ------------------------------------------------ TMA producer: packed weights ---
        if (lane == 0) {
            RingPos<C::SQ> ring;
            uint32_t issued = 0;
            bool ok_ = true;
            for (uint32_t t = cluster_id; t < ntiles && ok_; t += nclusters) {
                const int n0 = (int)(t / p.tiles_m) * BN + (int)rank * C::HB;
                for (uint32_t kb = 0; kb < p.nkb_main; ++kb) {
                    if (!mbar_wait(q_empty(ring.stage), ring.phase ^ 1u, abortp, C::POLL_PRODUCER)) {
                        fail(2, kb);
                        ok_ = false;
                        break;
                    }
                    mbar_expect_tx(q_full(ring.stage), C::Q_BYTES);
                    tma_load_2d(base + C::OFF_Q + ring.stage * C::Q_BYTES, &map_w, (int)(kb * 32), n0, q_full(ring.stage));
                    ring.advance();
                    ++issued;
                }
            }
            // Let every copy this thread issued land before the CTA may exit.
            for (uint32_t i = issued > (uint32_t)C::SQ ? issued - C::SQ : 0; i < issued; ++i) {
                const long long t0 = clock64();
                while (!mbar_try(q_full(i % C::SQ), (i / C::SQ) & 1u))
                    if (clock64() - t0 > 4000000000ll) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA) ---
        // Once per K block: wait for the stage, four MMAs, one commit. The whole warp
        // runs the loop converged and one elected lane issues the tcgen05
        // instructions: stage numbers and descriptors are then warp-uniform values,
        // which is what those instructions take, and the loop stays a few dozen
        // instructions (no division either). Whatever it spends between two blocks is
        // time the tensor cores can run dry.
        if (rank == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const uint32_t a_lo0 = umma_desc_lo(base + C::OFF_A), b_lo0 = umma_desc_lo(base + C::OFF_B);
            RingPos<C::SA> ring;
            uint32_t it = 0;
            bool ok_ = true;
            for (uint32_t t = cluster_id; t < ntiles && ok_; t += nclusters, ++it) {
                const uint32_t buf = it & 1u;
                if (!mbar_wait(acc_empty(buf), ((it >> 1) & 1u) ^ 1u, abortp)) {
                    if (lane == 0) fail(3, it);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d = tmem_base + buf * 256u;
                for (uint32_t kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(full(ring.stage), ring.phase, abortp)) {
                        if (lane == 0) fail(4, kb);
                        ok_ = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_lo = a_lo0 + ring.stage * (C::A_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + ring.stage * (C::B_BYTES >> 4);
                    tcgen05_mma_f16_pair_elect(d, a_lo, b_lo, idesc, kb);  // the tile's first MMA overwrites
#pragma unroll
                    for (uint32_t k4 = 1; k4 < 4; ++k4) tcgen05_mma_f16_pair_elect(d, a_lo + 2 * k4, b_lo + 2 * k4, idesc, 1u);
                    tcgen05_commit_pair_elect(empty(ring.stage));  // both CTAs' A and B stages are free once these MMAs have read them
                    ring.advance();
                }
                if (ok_) tcgen05_commit_pair_elect(acc_full(buf));
            }
            // Nothing may still be reading shared memory or writing TMEM when the pair winds down.
            tcgen05_commit_pair_local_elect(done_bar);
            const long long t0 = clock64();
            while (!mbar_try(done_bar, 0u))
                if (clock64() - t0 > 4000000000ll) break;
            __syncwarp();
        }
    } else if (warp == 3) {
        // idle: keeps the epilogue warps on TMEM lane quarters warp & 3
    } else if (warp < C::FIRST_DW) {
        // ------------------------------------------------ epilogue ---
        const uint32_t quarter = (uint32_t)warp & 3u;  // the TMEM lanes this warp may read
        uint32_t it = 0;
        for (uint32_t t = cluster_id; t < ntiles; t += nclusters, ++it) {
            const uint32_t buf = it & 1u;
            if (!mbar_wait(acc_full(buf), (it >> 1) & 1u, abortp, C::POLL_EPILOGUE)) {
                if (lane == 0) fail(5, it);
                break;
            }
            tcgen05_fence_after();
            const uint32_t m_base = ((t % p.tiles_m) * 2 + rank) * BM + quarter * 32;
            const uint32_t n0 = (t / p.tiles_m) * BN;
            const float rs = m_base + lane < p.M ? p.row_scale[m_base + lane] : 0.0f;
            const uint32_t stage = base + C::OFF_STAGE + quarter * 4096;
#pragma unroll 1
            for (uint32_t c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((quarter * 32u) << 16) + buf * 256u + c * 32u, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                store_block32_coalesced(p, r, stage, lane, m_base, n0 + c * 32, rs);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty(buf) + lead_delta);
        }
    } else {
        // ------------------------------------------------ dequant warps ---
        // Group g expands K blocks g, g + 2, ... of this CTA's BN/2 weight rows, two
        // threads per row: 16 packed bytes -> 32 f16 values each. The (scale, bias) word
        // of a block is fetched two blocks of this group ahead, right after a block was
        // handed over, so that no global load is still outstanding when the thread
        // reaches its next proxy fence (the fence waits for it).
        const uint32_t dw = (uint32_t)(warp - C::FIRST_DW);
        const uint32_t grp = dw / C::NDW;
        const uint32_t tg = (dw % C::NDW) * 32 + lane;
        const uint32_t r = tg >> 1, h = tg & 1u;  // weight row within this CTA's half; which 32 of the block's 64
        const uint32_t swz = (r & 7u) << 4;
        const uint32_t q_off = base + C::OFF_Q + r * 32 + h * 16, b_off = base + C::OFF_B + r * 128;
        bool ok_ = true;
        uint32_t it = 0;
        for (uint32_t t = cluster_id; t < ntiles && ok_; t += nclusters, ++it) {
            const uint32_t n = min((t / p.tiles_m) * BN + rank * C::HB + r, p.N - 1);  // rows past N repeat the last
            const uint32_t *sbrow = p.sb + (size_t)n * p.gpr;
            auto scale_word = [&](uint32_t kb) { return __ldg(sbrow + min((kb * 64 + h * 32) >> p.gshift, p.gpr - 1)); };
            uint32_t cur = scale_word(grp), nxt = scale_word(grp + C::NG);
            RingPos<C::SA> ring;   // stage of K block kb of this tile
            RingPos<C::SQ> qring;  // packed stage of that block
            ring.set(it * nkb + grp);
            qring.set(it * p.nkb_main + grp);
            for (uint32_t kb = grp; kb < nkb; kb += C::NG) {
                if (!mbar_wait(empty(ring.stage), ring.phase ^ 1u, abortp, C::POLL_DEQUANT)) {
                    if (lane == 0) fail(6, kb);
                    ok_ = false;
                    break;
                }
                const uint32_t brow = b_off + ring.stage * C::B_BYTES;
                if (kb < p.nkb_main) {
                    if (!mbar_wait(q_full(qring.stage), qring.phase, abortp, C::POLL_DEQUANT)) {
                        if (lane == 0) fail(7, kb);
                        ok_ = false;
                        break;
                    }
                    const uint4 w = lds128(q_off + qring.stage * C::Q_BYTES);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(q_empty(qring.stage));  // the packed stage may be refilled
                    qring.advance(C::NG);
                    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
                    expand_q4_words<4>(words, scale_h2(cur), brow, swz, 4 * h);
                } else {
                    expand_extra_chunks<4>(sbrow, kb - p.nkb_main, p.gpr, brow, swz, 4 * h);
                }
                // generic-proxy stores -> visible to the tensor cores' async-proxy reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(full(ring.stage) + lead_delta);
                ring.advance(C::NG);
                cur = nxt;
                if (kb + 2 * C::NG < p.nkb_main) nxt = scale_word(kb + 2 * C::NG);
            }
        }
    }

    // Neither CTA may leave, or give up its TMEM, while the other can still signal
    // its barriers or the pair's MMAs can still read its shared memory.
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

}  // namespace pf
}  // namespace tessl
