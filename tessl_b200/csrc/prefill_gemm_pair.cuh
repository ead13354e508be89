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
// Roles per CTA: warp 0 TMA producer, warp 1 TMEM allocation (+ MMA issue in the
// leader), warps 2-5 epilogue, then two groups of BN/64 dequant warps that take
// alternate K blocks. Every wait is bounded; on a timeout the status word is set
// and all roles fall through to the closing cluster barrier.
#pragma once
#include "prefill_common.cuh"

namespace tessl {
namespace pf {

template <int BN>
struct PairCfg {
    static constexpr int HB = BN / 2;                 // weight rows this CTA expands
    static constexpr int SA = 5;                      // stages of the (X tile, dequantized-W tile) ring
    static constexpr int SB = SA;                     // one ring: a K block's two operands are freed together
    static constexpr int SQ = 6;                      // packed-W stages
    static constexpr int NDW = HB / 32;               // dequant warps per group (one thread per weight row)
    static constexpr int NG = 2;                      // dequant groups; group g expands K blocks g, g + 2, ...
    static constexpr int THREADS = (6 + NG * NDW) * 32;
    static constexpr uint32_t A_BYTES = BM * BK * 2;  // 16 KiB
    static constexpr uint32_t Q_BYTES = HB * 32;
    static constexpr uint32_t B_BYTES = HB * BK * 2;
    static constexpr uint32_t OFF_A = 0;
    static constexpr uint32_t OFF_B = OFF_A + SA * A_BYTES;
    static constexpr uint32_t OFF_Q = OFF_B + SB * B_BYTES;
    static constexpr uint32_t OFF_BAR = OFF_Q + SQ * Q_BYTES;
    static constexpr int NBARS = 2 * SA + 2 * SQ + 2 * SB + 4 + 1;
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
    auto a_full = [&](int s) { return bar0 + 8 * s; };                                      // leader's is used
    auto a_empty = [&](int s) { return bar0 + 8 * (C::SA + s); };                           // both; frees A and B
    auto q_full = [&](int s) { return bar0 + 8 * (2 * C::SA + s); };                        // CTA-local
    auto q_empty = [&](int s) { return bar0 + 8 * (2 * C::SA + C::SQ + s); };               // CTA-local
    auto b_full = [&](int s) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + s); };            // leader's is used
    auto b_empty = [&](int s) { return a_empty(s); };  // stage s of both operands is released by one commit
    auto acc_full = [&](int b) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + 2 * C::SB + b); };       // both
    auto acc_empty = [&](int b) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + 2 * C::SB + 2 + b); };  // leader's
    const uint32_t done_bar = bar0 + 8 * (2 * C::SA + 2 * C::SQ + 2 * C::SB + 4);
    // The leader's barrier block as seen from this CTA (its own block when this CTA leads).
    const uint32_t lead_delta = map_to_cta(bar0, 0) - bar0;

    const uint32_t nkb = p.nkb_main + p.nkb_extra;
    const uint32_t ntiles = p.tiles_m * p.tiles_n;  // pair tiles: tiles_m counts 256-row blocks
    const uint32_t cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::SA; ++s) mbar_init(a_full(s), 1), mbar_init(a_empty(s), 1);
        for (int s = 0; s < C::SQ; ++s) mbar_init(q_full(s), 1), mbar_init(q_empty(s), C::NDW);
        for (int s = 0; s < C::SB; ++s) mbar_init(b_full(s), 2 * C::NDW);
        for (int b = 0; b < 2; ++b) mbar_init(acc_full(b), 1), mbar_init(acc_empty(b), 8);
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
#ifdef TESSL_GEMM_TIMING
    long long tacc[6] = {0, 0, 0, 0, 0, 0};
    const long long tstart = clock64();
    long long tlast = tstart;
#endif

    if (warp == 0) {
        // ------------------------------------------------ TMA producer ---
        if (lane == 0) {
            uint32_t ia = 0, iq = 0;  // running stage counters
            bool ok_ = true;
            for (uint32_t t = cluster_id; t < ntiles && ok_; t += nclusters) {
                const int m0 = (int)((t % p.tiles_m) * 2 + rank) * BM;
                const int n0 = (int)(t / p.tiles_m) * BN + (int)rank * C::HB;
                for (uint32_t kb = 0; kb < nkb; ++kb) {
                    const uint32_t sa = ia % C::SA;
                    if (!mbar_wait(a_empty(sa), ((ia / C::SA) & 1u) ^ 1u, abortp)) {
                        fail(1, kb);
                        ok_ = false;
                        break;
                    }
                    TSTAMP(0);  // wait a_empty
                    // The leader expects both CTAs' tiles on its barrier; either CTA's bytes may land first.
                    if (rank == 0) mbar_expect_tx(a_full(sa), 2 * C::A_BYTES);
                    tma_load_2d_pair(base + C::OFF_A + sa * C::A_BYTES, &map_a, (int)(kb * BK), m0,
                                     a_full(sa) + lead_delta);
                    ++ia;
                    TSTAMP(1);  // issue A
                    if (kb < p.nkb_main) {
                        const uint32_t sq = iq % C::SQ;
                        if (!mbar_wait(q_empty(sq), ((iq / C::SQ) & 1u) ^ 1u, abortp)) {
                            fail(2, kb);
                            ok_ = false;
                            break;
                        }
                        TSTAMP(2);  // wait q_empty
                        mbar_expect_tx(q_full(sq), C::Q_BYTES);
                        tma_load_2d(base + C::OFF_Q + sq * C::Q_BYTES, &map_w, (int)(kb * 32), n0, q_full(sq));
                        ++iq;
                        TSTAMP(3);  // issue Q
                    }
                }
            }
            // Let every packed-weight copy this thread issued land before the CTA may exit; the
            // activation copies are covered by the leader's wait for its last MMA below.
            for (uint32_t i = iq > (uint32_t)C::SQ ? iq - C::SQ : 0; i < iq; ++i) {
                const long long t0 = clock64();
                while (!mbar_try(q_full(i % C::SQ), (i / C::SQ) & 1u))
                    if (clock64() - t0 > 4000000000ll) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA) ---
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            uint32_t ia = 0, ib = 0, it = 0;
            bool ok_ = true;
            for (uint32_t t = cluster_id; t < ntiles && ok_; t += nclusters, ++it) {
                const uint32_t buf = it & 1u;
                if (!mbar_wait(acc_empty(buf), ((it >> 1) & 1u) ^ 1u, abortp)) {
                    fail(3, it);
                    break;
                }
                tcgen05_fence_after();
                TSTAMP(0);  // wait acc_empty
                const uint32_t d = tmem_base + buf * 256u;
                for (uint32_t kb = 0; kb < nkb; ++kb) {
                    const uint32_t sa = ia % C::SA, sb = ib % C::SB;
                    if (!mbar_wait(a_full(sa), (ia / C::SA) & 1u, abortp)) {
                        fail(4, kb);
                        ok_ = false;
                        break;
                    }
                    TSTAMP(1);  // wait a_full
                    if (!mbar_wait(b_full(sb), (ib / C::SB) & 1u, abortp)) {
                        fail(4, kb);
                        ok_ = false;
                        break;
                    }
                    TSTAMP(2);  // wait b_full
                    tcgen05_fence_after();
                    const uint64_t ad = umma_desc(base + C::OFF_A + sa * C::A_BYTES);
                    const uint64_t bd = umma_desc(base + C::OFF_B + sb * C::B_BYTES);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; ++k4)
                        tcgen05_mma_f16_pair(d, ad + 2 * k4, bd + 2 * k4, idesc, (kb | k4) != 0 ? 1u : 0u);
                    tcgen05_commit_pair(a_empty(sa));  // both CTAs' A and B stages are free once these MMAs have read them
                    ++ia, ++ib;
                    TSTAMP(3);  // issue MMAs and commits
                }
                if (ok_) tcgen05_commit_pair(acc_full(buf));
            }
            // Nothing may still be reading shared memory or writing TMEM when the pair winds down.
            tcgen05_commit_pair_local(done_bar);
            const long long t0 = clock64();
            while (!mbar_try(done_bar, 0u))
                if (clock64() - t0 > 4000000000ll) break;
        }
    } else if (warp < 6) {
        // ------------------------------------------------ epilogue ---
        const uint32_t quarter = (uint32_t)warp & 3u;  // the TMEM lanes this warp may read
        uint32_t it = 0;
        for (uint32_t t = cluster_id; t < ntiles; t += nclusters, ++it) {
            const uint32_t buf = it & 1u;
            if (!mbar_wait(acc_full(buf), (it >> 1) & 1u, abortp)) {
                if (lane == 0) fail(5, it);
                break;
            }
            tcgen05_fence_after();
            TSTAMP(0);  // wait acc_full
            const uint32_t m = ((t % p.tiles_m) * 2 + rank) * BM + quarter * 32 + lane;
            const uint32_t n0 = (t / p.tiles_m) * BN;
            const float rs = m < p.M ? p.row_scale[m] : 0.0f;
#pragma unroll 1
            for (uint32_t c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((quarter * 32u) << 16) + buf * 256u + c * 32u, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                store_row32(p, r, m, n0 + c * 32, rs);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty(buf) + lead_delta);
            TSTAMP(1);  // drain the accumulator
        }
    } else {
        // ------------------------------------------------ dequant warps ---
        // Group g expands K blocks g, g + 2, ... of this CTA's BN/2 weight rows. The
        // (scale, bias) words of a block are fetched two blocks of this group ahead,
        // right after a block was handed over, so that no global load is still
        // outstanding when the thread reaches its next proxy fence (the fence waits for it).
        const uint32_t dw = (uint32_t)(warp - 6);
        const uint32_t grp = dw / C::NDW;
        const uint32_t r = (dw % C::NDW) * 32 + lane;  // weight row within this CTA's half
        const uint32_t swz = (r & 7u) << 4;
        bool ok_ = true;
        uint32_t it = 0;
        for (uint32_t t = cluster_id; t < ntiles && ok_; t += nclusters, ++it) {
            const uint32_t n = min((t / p.tiles_m) * BN + rank * C::HB + r, p.N - 1);  // rows past N repeat the last
            const uint32_t *sbrow = p.sb + (size_t)n * p.gpr;
            auto scale_word = [&](uint32_t kb, int h) {
                return __ldg(sbrow + min((kb * 64 + h * 32) >> p.gshift, p.gpr - 1));
            };
            uint32_t cur[2] = {scale_word(grp, 0), scale_word(grp, 1)};
            uint32_t nxt[2] = {scale_word(grp + C::NG, 0), scale_word(grp + C::NG, 1)};
            for (uint32_t kb = grp; kb < nkb; kb += C::NG) {
                const uint32_t ib = it * nkb + kb;                          // global K-block index
                const uint32_t iq = it * p.nkb_main + min(kb, p.nkb_main);  // global packed-stage index
                const uint32_t sb = ib % C::SB;
                if (!mbar_wait(b_empty(sb), ((ib / C::SB) & 1u) ^ 1u, abortp)) {
                    if (lane == 0) fail(6, kb);
                    ok_ = false;
                    break;
                }
                TSTAMP(0);  // wait b_empty
                const uint32_t brow = base + C::OFF_B + sb * C::B_BYTES + r * 128;
                if (kb < p.nkb_main) {
                    const uint32_t sq = iq % C::SQ;
                    if (!mbar_wait(q_full(sq), (iq / C::SQ) & 1u, abortp)) {
                        if (lane == 0) fail(7, kb);
                        ok_ = false;
                        break;
                    }
                    TSTAMP(1);  // wait q_full
                    const uint32_t qrow = base + C::OFF_Q + sq * C::Q_BYTES + r * 32;
                    const uint4 w0 = lds128(qrow), w1 = lds128(qrow + 16);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(q_empty(sq));  // the packed stage may be refilled
                    TSTAMP(2);  // read the packed row
                    const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                    const uint32_t s2[2] = {scale_h2(cur[0]), scale_h2(cur[1])};
                    expand_q4_block(words, s2, brow, swz);
                } else {
                    expand_extra_block(sbrow, kb - p.nkb_main, p.gpr, brow, swz);
                }
                TSTAMP(3);  // expand and store
                // generic-proxy stores -> visible to the tensor cores' async-proxy reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                TSTAMP(4);  // proxy fence
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(b_full(sb) + lead_delta);
                cur[0] = nxt[0], cur[1] = nxt[1];
                if (kb + 2 * C::NG < p.nkb_main)
                    nxt[0] = scale_word(kb + 2 * C::NG, 0), nxt[1] = scale_word(kb + 2 * C::NG, 1);
                TSTAMP(5);  // hand over, prefetch
            }
        }
    }

#ifdef TESSL_GEMM_TIMING
    if (p.timing && lane == 0) {
        // rows of 8 slots: 0 producer, 1 MMA issuer, 2 epilogue warp 2, 3 dequant warp 6; slot 7 = role's total
        const int role = warp == 0 ? 0 : warp == 1 ? 1 : warp == 2 ? 2 : warp == 6 ? 3 : -1;
        if (role >= 0) {
            long long *o = p.timing + (size_t)blockIdx.x * 32 + role * 8;
            for (int i = 0; i < 6; ++i) o[i] = tacc[i];
            o[7] = clock64() - tstart;
        }
    }
#endif
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
