// MLX Q4 prefill GEMM on the tcgen05 tensor cores:
//
//     Y[M, N] = X[M, K] (bf16) . W[N, K]^T,   W = scale * q + bias per group of G along K
//
// the replacement for the reference's `nn::gemm_q4_mlx_tensorops`
// (src/nn.rs:4683-4757; kernels/gemm_q4_mlx_tensorops.metal in the reference
// project). The reference keeps the integer nibbles exact in its matrix unit and
// folds the affine in f32; rounding the dequantized weight to bf16 (8 significand
// bits) would not stay inside the stated output tolerance, so this kernel keeps
// the products exact too, with f16 operands:
//
//     W = s * (q - 8) + (b + 8 s)
//
//   * s * (q - 8) has at most 8 + 3 significand bits: exact in f16 (for
//     2^-17 <= |s| <= 8188; real MLX scales are 1e-4 .. 1e-1). It is the B operand,
//     produced in shared memory from the packed nibbles.
//   * X is converted bf16 -> f16 once per call by a small pre-pass, after an exact
//     per-row power-of-two rescale so any finite bf16 row fits f16's range; the
//     scale is undone in the epilogue. That is the A operand.
//   * The remaining rank-K/G term sum_g xsum[m, g] * (b + 8 s)[n, g] rides along
//     as extra K columns: the pre-pass appends, per group, the f32 group sum of x
//     split into three f16 pieces (h1, h2, h3, h1) and the dequant warps emit
//     (c1, c1, c1, c2) with c1 + c2 the two-piece f16 split of b + 8 s. Four
//     extra columns per group, ~6% more MMA work at G = 64.
//
// Every product is exact and accumulation is f32 in TMEM, so the result obeys
// the reference's own bound gamma_t * S (tests/gemm_q4_mlx_tensorops.rs:11-21 of
// the reference project).
//
// Structure (one CTA per SM, persistent over 128 x BN output tiles):
//   warp 0      TMA producer: X tile (128 x 64 f16, 128B swizzle) and packed W
//               tile (BN rows x 32 bytes) per 64-wide K block, plain
//               cp.async.bulk.tensor loads (no multicast).
//   warp 1      allocates TMEM (512 columns = two BN-wide f32 accumulators) and
//               issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BN,
//               K = 16, four per K block), committing to mbarriers.
//   warps 2-5   epilogue: tcgen05.ld of the finished accumulator, row scale,
//               stores; overlaps the next tile's main loop.
//   warps 6..   BN/32 dequant warps, one thread per weight row: 32 packed bytes
//               from shared memory -> 64 f16 values s * (q - 8) written in the
//               128B-swizzled K-major layout the MMA descriptor expects.
// All mbarrier waits are bounded (see q4_gemv_tma.cuh); on a timeout the status
// word is set, every role leaves its loops and TMEM is released.
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "prefill_common.cuh"
#include "prefill_gemm_pair.cuh"

namespace tessl {
namespace {

using namespace pf;
using nn::OutKind;
using nn::OUT_BF16;

// ------------------------------------------------------- activation pre-pass ---

/// One block per X row: finds the row's exponent, writes the row as f16 scaled by
/// an exact power of two into the augmented A matrix (K padded to 64, elements of
/// every 8-chunk in the order 0,4,1,5,2,6,3,7 that the nibble-pair dequant
/// produces on the B side), then the per-group sums as (h1, h2, h3, h1) f16
/// quadruples, then zero padding. a_aug is [M, K_aug] row-major.
__global__ void __launch_bounds__(256) x_prepare_kernel(const uint16_t *x, __half *a_aug, float *row_scale, uint32_t K,
                                                        uint32_t K64, uint32_t K_aug, uint32_t gshift)
{
    const uint32_t m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint16_t *xrow = x + (size_t)m * K;
    __half *arow = a_aug + (size_t)m * K_aug;
    __shared__ uint32_t red[8];
    __shared__ float s_down;

    // pass 1: largest magnitude (bf16 bit patterns order like integers); Inf/NaN disable the rescale
    uint32_t amax = 0;
    for (uint32_t ch = tid; ch < K / 8; ch += 256) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(xrow) + ch);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) amax = max(amax, max(w[j] & 0x7fffu, (w[j] >> 16) & 0x7fffu));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    if (tid == 0) {
        uint32_t a = 0;
        for (int i = 0; i < 8; ++i) a = max(a, red[i]);
        int sh = 0;
        if (a != 0 && a < 0x7f80u) {
            const int e = (int)(a >> 7) - 127;  // floor(log2 max|x|)
            // Bring the row maximum to [2^14 / G, 2^15 / G): every element and every
            // group sum (at most G times the maximum) then fits f16.
            sh = min(max(e - 14 + (int)gshift, -126), 126);
        }
        s_down = __int_as_float((127 - sh) << 23);
        row_scale[m] = __int_as_float((127 + sh) << 23);
    }
    __syncthreads();
    const float down = s_down;

    // pass 2: convert, permute, group sums
    const uint32_t gsize8 = (1u << gshift) / 8;  // 8-element chunks per group: 4, 8 or 16
    const uint32_t gpr = K >> gshift;
    for (uint32_t base = 0; base < K64 / 8; base += 256) {
        const uint32_t ch = base + tid;
        float f[8];
        if (ch * 8 < K) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(xrow) + ch);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[2 * j] = __uint_as_float(w[j] << 16) * down;
                f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u) * down;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = 0.0f;
        }
        __half h[8];
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            h[j] = __float2half_rn(f[j]);
            sum += __half2float(h[j]);  // the group sum is over the values the MMA will see
        }
        if (ch < K64 / 8) {
            uint4 o;
            o.x = pack_h2(h[0], h[4]), o.y = pack_h2(h[1], h[5]), o.z = pack_h2(h[2], h[6]), o.w = pack_h2(h[3], h[7]);
            reinterpret_cast<uint4 *>(arow)[ch] = o;
        }
        for (uint32_t o = gsize8 / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const uint32_t g = ch / gsize8;
        if ((ch % gsize8) == 0 && g < gpr) {
            const __half h1 = __float2half_rn(sum);
            const float r1 = sum - __half2float(h1);
            const __half h2 = __float2half_rn(r1);
            const __half h3 = __float2half_rn(r1 - __half2float(h2));
            uint2 q;
            q.x = pack_h2(h1, h2), q.y = pack_h2(h3, h1);
            *reinterpret_cast<uint2 *>(arow + K64 + 4 * g) = q;
        }
    }
    // pass 3: zero the unused tail of the extra columns
    for (uint32_t i = 4 * gpr + tid; i < K_aug - K64; i += 256) arow[K64 + i] = __float2half_rn(0.0f);
}

// ------------------------------------------------------------------ the GEMM ---

template <int BN>
struct Cfg {
    static constexpr int SA = 4;                      // X-tile stages
    static constexpr int SQ = 4;                      // packed-W stages
    static constexpr int SB = BN == 256 ? 3 : 4;      // dequantized-W stages
    static constexpr int NDW = BN / 32;               // dequant warps
    static constexpr int THREADS = (6 + NDW) * 32;
    static constexpr uint32_t A_BYTES = BM * BK * 2;  // 16 KiB
    static constexpr uint32_t Q_BYTES = BN * 32;
    static constexpr uint32_t B_BYTES = BN * BK * 2;
    static constexpr uint32_t OFF_A = 0;
    static constexpr uint32_t OFF_B = OFF_A + SA * A_BYTES;
    static constexpr uint32_t OFF_Q = OFF_B + SB * B_BYTES;
    static constexpr uint32_t OFF_BAR = OFF_Q + SQ * Q_BYTES;
    static constexpr int NBARS = 2 * SA + 2 * SQ + 2 * SB + 4 + 1;
    static constexpr uint32_t SMEM = OFF_BAR + NBARS * 8 + 1024;  // + slack to align the base to 1 KiB
};

template <int BN>
__global__ void __launch_bounds__(Cfg<BN>::THREADS, 1)
    q4_prefill_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                           const GemmParams p)
{
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = base + C::OFF_BAR;
    auto a_full = [&](int s) { return bar0 + 8 * s; };
    auto a_empty = [&](int s) { return bar0 + 8 * (C::SA + s); };
    auto q_full = [&](int s) { return bar0 + 8 * (2 * C::SA + s); };
    auto q_empty = [&](int s) { return bar0 + 8 * (2 * C::SA + C::SQ + s); };
    auto b_full = [&](int s) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + s); };
    auto b_empty = [&](int s) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + C::SB + s); };
    auto acc_full = [&](int b) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + 2 * C::SB + b); };
    auto acc_empty = [&](int b) { return bar0 + 8 * (2 * C::SA + 2 * C::SQ + 2 * C::SB + 2 + b); };
    const uint32_t done_bar = bar0 + 8 * (C::NBARS - 1);

    const uint32_t nkb = p.nkb_main + p.nkb_extra;
    const uint32_t ntiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::SA; ++s) mbar_init(a_full(s), 1), mbar_init(a_empty(s), 1);
        for (int s = 0; s < C::SQ; ++s) mbar_init(q_full(s), 1), mbar_init(q_empty(s), C::NDW);
        for (int s = 0; s < C::SB; ++s) mbar_init(b_full(s), C::NDW), mbar_init(b_empty(s), 1);
        for (int b = 0; b < 2; ++b) mbar_init(acc_full(b), 1), mbar_init(acc_empty(b), 4);
        mbar_init(done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;
    auto fail = [&](uint32_t role, uint32_t where) {
        *abortp = 1;
        *(volatile uint32_t *)p.status = (role << 24) | (where & 0xffffffu);
    };

    if (warp == 0) {
        // ------------------------------------------------ TMA producer ---
        if (lane == 0) {
            uint32_t ia = 0, iq = 0;  // running stage counters
            bool ok_ = true;
            for (uint32_t t = blockIdx.x; t < ntiles && ok_; t += gridDim.x) {
                const int m0 = (int)(t % p.tiles_m) * BM, n0 = (int)(t / p.tiles_m) * BN;
                for (uint32_t kb = 0; kb < nkb; ++kb) {
                    const uint32_t sa = ia % C::SA;
                    if (!mbar_wait(a_empty(sa), ((ia / C::SA) & 1u) ^ 1u, abortp)) {
                        fail(1, kb);
                        ok_ = false;
                        break;
                    }
                    mbar_expect_tx(a_full(sa), C::A_BYTES);
                    tma_load_2d(base + C::OFF_A + sa * C::A_BYTES, &map_a, (int)(kb * BK), m0, a_full(sa));
                    ++ia;
                    if (kb < p.nkb_main) {
                        const uint32_t sq = iq % C::SQ;
                        if (!mbar_wait(q_empty(sq), ((iq / C::SQ) & 1u) ^ 1u, abortp)) {
                            fail(2, kb);
                            ok_ = false;
                            break;
                        }
                        mbar_expect_tx(q_full(sq), C::Q_BYTES);
                        tma_load_2d(base + C::OFF_Q + sq * C::Q_BYTES, &map_w, (int)(kb * 32), n0, q_full(sq));
                        ++iq;
                    }
                }
            }
            // Let every copy this thread issued land before the CTA may exit.
            for (uint32_t i = ia > (uint32_t)C::SA ? ia - C::SA : 0; i < ia; ++i) {
                const long long t0 = clock64();
                while (!mbar_try(a_full(i % C::SA), (i / C::SA) & 1u))
                    if (clock64() - t0 > 4000000000ll) break;
            }
            for (uint32_t i = iq > (uint32_t)C::SQ ? iq - C::SQ : 0; i < iq; ++i) {
                const long long t0 = clock64();
                while (!mbar_try(q_full(i % C::SQ), (i / C::SQ) & 1u))
                    if (clock64() - t0 > 4000000000ll) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer ---
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t ia = 0, ib = 0, it = 0;
            bool ok_ = true;
            for (uint32_t t = blockIdx.x; t < ntiles && ok_; t += gridDim.x, ++it) {
                const uint32_t buf = it & 1u;
                if (!mbar_wait(acc_empty(buf), ((it >> 1) & 1u) ^ 1u, abortp)) {
                    fail(3, it);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d = tmem_base + buf * 256u;
                for (uint32_t kb = 0; kb < nkb; ++kb) {
                    const uint32_t sa = ia % C::SA, sb = ib % C::SB;
                    if (!mbar_wait(a_full(sa), (ia / C::SA) & 1u, abortp) ||
                        !mbar_wait(b_full(sb), (ib / C::SB) & 1u, abortp)) {
                        fail(4, kb);
                        ok_ = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint64_t ad = umma_desc(base + C::OFF_A + sa * C::A_BYTES);
                    const uint64_t bd = umma_desc(base + C::OFF_B + sb * C::B_BYTES);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; ++k4)
                        tcgen05_mma_f16(d, ad + 2 * k4, bd + 2 * k4, idesc, (kb | k4) != 0 ? 1u : 0u);
                    tcgen05_commit(a_empty(sa));  // both stages are free once these MMAs have read them
                    tcgen05_commit(b_empty(sb));
                    ++ia, ++ib;
                }
                if (ok_) tcgen05_commit(acc_full(buf));
            }
            // Nothing may still be writing TMEM when it is released below.
            tcgen05_commit(done_bar);
            const long long t0 = clock64();
            while (!mbar_try(done_bar, 0u))
                if (clock64() - t0 > 4000000000ll) break;
        }
    } else if (warp < 6) {
        // ------------------------------------------------ epilogue ---
        const uint32_t quarter = (uint32_t)warp & 3u;  // the TMEM lanes this warp may read
        uint32_t it = 0;
        for (uint32_t t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
            const uint32_t buf = it & 1u;
            if (!mbar_wait(acc_full(buf), (it >> 1) & 1u, abortp)) {
                if (lane == 0) fail(5, it);
                break;
            }
            tcgen05_fence_after();
            const uint32_t m = (t % p.tiles_m) * BM + quarter * 32 + lane;
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
            if (lane == 0) mbar_arrive(acc_empty(buf));
        }
    } else {
        // ------------------------------------------------ dequant warps ---
        const uint32_t r = (uint32_t)(warp - 6) * 32 + lane;  // weight row within the tile
        const uint32_t swz = (r & 7u) << 4;
        uint32_t iq = 0, ib = 0;
        bool ok_ = true;
        for (uint32_t t = blockIdx.x; t < ntiles && ok_; t += gridDim.x) {
            const uint32_t n = min((t / p.tiles_m) * BN + r, p.N - 1);  // rows past N repeat the last row
            const uint32_t *sbrow = p.sb + (size_t)n * p.gpr;
            for (uint32_t kb = 0; kb < nkb; ++kb) {
                const uint32_t sb = ib % C::SB;
                if (!mbar_wait(b_empty(sb), ((ib / C::SB) & 1u) ^ 1u, abortp)) {
                    if (lane == 0) fail(6, kb);
                    ok_ = false;
                    break;
                }
                const uint32_t brow = base + C::OFF_B + sb * C::B_BYTES + r * 128;
                if (kb < p.nkb_main) {
                    const uint32_t sq = iq % C::SQ;
                    if (!mbar_wait(q_full(sq), (iq / C::SQ) & 1u, abortp)) {
                        if (lane == 0) fail(7, kb);
                        ok_ = false;
                        break;
                    }
                    const uint32_t qrow = base + C::OFF_Q + sq * C::Q_BYTES + r * 32;
                    const uint4 w0 = lds128(qrow), w1 = lds128(qrow + 16);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(q_empty(sq));  // the packed stage may be refilled
                    ++iq;
                    const uint32_t lo[4] = {w0.x, w0.y, w0.z, w0.w}, hi[4] = {w1.x, w1.y, w1.z, w1.w};
                    const uint32_t g0 = min((kb * 64) >> p.gshift, p.gpr - 1);
                    const uint32_t g1 = min((kb * 64 + 32) >> p.gshift, p.gpr - 1);
                    expand_q4_words<4>(lo, scale_h2(__ldg(sbrow + g0)), brow, swz, 0);
                    expand_q4_words<4>(hi, scale_h2(__ldg(sbrow + g1)), brow, swz, 4);
                } else {
                    expand_extra_chunks<8>(sbrow, kb - p.nkb_main, p.gpr, brow, swz, 0);
                }
                // generic-proxy stores -> visible to the tensor core's async-proxy reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(b_full(sb));
                ++ib;
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------- host ---

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

Result tensormap_encoder(TesslRuntime *rt, EncodeTiled *out)
{
    if (!rt->tensormap_encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            cudaGetLastError();
            return "gemm_q4_mlx_tensorops: the driver does not export cuTensorMapEncodeTiled";
        }
        rt->tensormap_encode = fn;
    }
    *out = reinterpret_cast<EncodeTiled>(rt->tensormap_encode);
    return ok();
}

Result make_map_2d(EncodeTiled enc, CUtensorMap *map, CUtensorMapDataType dt, void *ptr, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz)
{
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, dt, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fmt("gemm_q4_mlx_tensorops: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return ok();
}

template <int BN>
Result launch_gemm(TesslRuntime *rt, const CUtensorMap &ma, const CUtensorMap &mw, GemmParams p)
{
    using C = Cfg<BN>;
    auto kernel = q4_prefill_gemm_kernel<BN>;
    TESSL_TRY(smem_opt_in(rt, reinterpret_cast<const void *>(kernel), C::SMEM, "gemm_q4_mlx_tensorops: shared memory opt-in"));
    const uint32_t tiles = p.tiles_m * p.tiles_n;
    const uint32_t grid = std::min<uint32_t>(tiles, (uint32_t)rt->sm_count);
    kernel<<<grid, C::THREADS, C::SMEM, rt->stream>>>(ma, mw, p);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "gemm_q4_mlx_tensorops launch");
}

/// The CTA-pair kernel: one cluster of two CTAs per pair of SMs, persistent over 256 x BN tiles.
template <int BN>
Result launch_gemm_pair(TesslRuntime *rt, const CUtensorMap &ma, const CUtensorMap &mw, GemmParams p)
{
    using C = PairCfg<BN>;
    auto kernel = q4_prefill_gemm_pair_kernel<BN>;
    TESSL_TRY(smem_opt_in(rt, reinterpret_cast<const void *>(kernel), C::SMEM, "gemm_q4_mlx_tensorops: shared memory opt-in"));
    const uint32_t tiles = p.tiles_m * p.tiles_n;
    const uint32_t clusters = std::min<uint32_t>(tiles, (uint32_t)rt->sm_count / 2);
    kernel<<<2 * clusters, C::THREADS, C::SMEM, rt->stream>>>(ma, mw, p);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "gemm_q4_mlx_tensorops launch");
}

/// Shapes and scratch layout of one prefill GEMM call.
struct PrefillPlan {
    uint32_t n, k, groups, gshift, nkb_main, nkb_extra, k64, k_aug;
    size_t a_bytes;  // augmented f16 activations [m, k_aug], rounded up to 256 bytes
    size_t need;     // a_bytes + m row scales
};

/// Argument checks shared by the allocating and the non-allocating entry, in the
/// reference's order (src/nn.rs:4697-4740 of the reference project). `*empty` is
/// set when there is nothing to compute.
Result prefill_validate(const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                        const TesslQuantShape &shape, uint32_t m, OutKind out, PrefillPlan *plan, bool *empty)
{
    const char *what = "gemm_q4_mlx_tensorops";
    TESSL_TRY(quant_shape_validate(shape, what));
    if (shape.group_size != 32 && shape.group_size != 64 && shape.group_size != 128) {
        return fmt("%s: group_size %u is not one of [32, 64, 128]; the matmul2d descriptor's K is the group, so each "
                   "size is its own entry point",
                   what, shape.group_size);
    }
    if (shape.cols == 0) return fmt("%s: cols must be non-zero", what);
    const uint32_t n = shape.rows, k = shape.cols, groups = k / shape.group_size;
    // The reference kernel's int32 extents; checked before any buffer length so an
    // oversize shape is named as such (src/nn.rs:4712-4727 of the reference project).
    TESSL_TRY(require_i32_extent(elems(m, k), "gemm_q4_mlx_tensorops x (m * cols)"));
    TESSL_TRY(require_i32_extent(elems(n, k), "gemm_q4_mlx_tensorops weights (rows * cols 4-bit elements)"));
    TESSL_TRY(require_i32_extent(elems(m, n), "gemm_q4_mlx_tensorops y (m * rows)"));
    TESSL_TRY(require_i32_extent(elems(n, groups), "gemm_q4_mlx_tensorops scale/bias pairs (rows * groups)"));
    TESSL_TRY(q4_bank_validate(bank, shape, what));
    TESSL_TRY(require(x_bf16, elems(m, k), 2, std::string(what) + " x_bf16"));
    TESSL_TRY(require(y, elems(m, n), out == OUT_BF16 ? 2 : 4, std::string(what) + " y"));
    const Named writes[] = {{"y", &y}};
    const Named reads[] = {{"packed", &bank.packed}, {"scales_biases", &bank.scales_biases}, {"x_bf16", &x_bf16}};
    TESSL_TRY(require_disjoint_writes(what, writes, 1, reads, 3));
    *empty = m == 0 || n == 0;
    if (*empty) return ok();
    TESSL_TRY(require_aligned16(bank.packed, std::string(what) + " packed"));
    TESSL_TRY(require_aligned16(x_bf16, std::string(what) + " x_bf16"));
    TESSL_TRY(require_aligned16(y, std::string(what) + " y"));
    if (((uintptr_t)bank.scales_biases.ptr & 3u) != 0)
        return fmt("%s scales_biases: device pointer must be 4-byte aligned", what);

    PrefillPlan pl{};
    pl.n = n, pl.k = k, pl.groups = groups;
    while ((1u << pl.gshift) < shape.group_size) ++pl.gshift;
    pl.nkb_main = (k + BK - 1) / BK;
    pl.nkb_extra = (4 * groups + BK - 1) / BK;
    pl.k64 = pl.nkb_main * BK, pl.k_aug = (pl.nkb_main + pl.nkb_extra) * BK;
    pl.a_bytes = ((size_t)m * pl.k_aug * 2 + 255) & ~(size_t)255;
    pl.need = pl.a_bytes + (size_t)m * 4;
    *plan = pl;
    return ok();
}

/// The pair kernel's 256-row tile is half padding for m <= 128, but each CTA still expands only half of
/// the weight rows and it has the better pipeline: measured 34.6 us against the single-CTA kernel's 48.9 us
/// at m = 16 .. 64, N = 12288, K = 4096. So the pair kernel runs for every m; the single-CTA kernel is
/// what a GPU with one SM, or `tessl_runtime_set_prefill_tile(rt, bn, 0)`, selects.

/// Tile width with the least estimated time: waves of tiles x the cost of one tile's K block.
int pick_tile_width(uint64_t tiles_m, uint32_t n, uint32_t slots)
{
    int best_bn = 256;
    uint64_t best_cost = ~0ull;
    for (int bn : {256, 192, 128}) {
        const uint64_t tiles = tiles_m * ((n + bn - 1) / bn);
        const uint64_t waves = (tiles + slots - 1) / slots;
        // a K block costs a fixed part (measured: about 320 columns' worth) plus a part proportional to the width
        const uint64_t cost = waves * (uint64_t)(bn + 320);
        if (cost < best_cost) best_cost = cost, best_bn = bn;
    }
    return best_bn;
}

/// Pre-pass and GEMM of a validated call; `scratch` holds `plan.need` bytes.
Result prefill_launch(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y, uint32_t m,
                      OutKind out, const PrefillPlan &pl, void *scratch)
{
    __half *a_aug = static_cast<__half *>(scratch);
    float *row_scale = reinterpret_cast<float *>(static_cast<char *>(scratch) + pl.a_bytes);
    x_prepare_kernel<<<m, 256, 0, rt->stream>>>(static_cast<const uint16_t *>(x_bf16.ptr), a_aug, row_scale, pl.k, pl.k64,
                                                pl.k_aug, pl.gshift);
    rt->dispatch_count += 1;
    TESSL_TRY(cuda_check(rt, cudaGetLastError(), "gemm_q4_mlx_tensorops pre-pass launch"));

    const bool pair = rt->sm_count >= 2 && rt->prefill_force_pair != 0;
    const uint32_t tiles_m = pair ? (m + 2 * BM - 1) / (2 * BM) : (m + BM - 1) / BM;
    const int bn = rt->prefill_force_bn
                       ? rt->prefill_force_bn
                       : pick_tile_width(tiles_m, pl.n, pair ? (uint32_t)rt->sm_count / 2 : (uint32_t)rt->sm_count);
    rt->prefill_last_bn = bn, rt->prefill_last_pair = pair ? 1 : 0;

    EncodeTiled enc = nullptr;
    TESSL_TRY(tensormap_encoder(rt, &enc));
    CUtensorMap ma, mw;
    TESSL_TRY(make_map_2d(enc, &ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a_aug, pl.k_aug, m, (uint64_t)pl.k_aug * 2, BK, BM,
                          CU_TENSOR_MAP_SWIZZLE_128B));
    // Packed weights: 32 bytes of BN rows (single CTA) or of this CTA's BN/2 rows (pair) per K block.
    TESSL_TRY(make_map_2d(enc, &mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, bank.packed.ptr, pl.k / 2, pl.n, pl.k / 2, 32,
                          (uint32_t)(pair ? bn / 2 : bn), CU_TENSOR_MAP_SWIZZLE_NONE));

    GemmParams p{};
    p.sb = static_cast<const uint32_t *>(bank.scales_biases.ptr);
    p.row_scale = row_scale;
    p.y = y.ptr;
    p.M = m, p.N = pl.n, p.K = pl.k;
    p.gshift = pl.gshift, p.gpr = pl.groups;
    p.nkb_main = pl.nkb_main, p.nkb_extra = pl.nkb_extra;
    p.tiles_m = tiles_m;
    p.tiles_n = (pl.n + bn - 1) / bn;
    p.out_bf16 = out == OUT_BF16;
    p.status = rt->status_dev;
    if (pair) {
        if (bn == 256) return launch_gemm_pair<256>(rt, ma, mw, p);
        if (bn == 192) return launch_gemm_pair<192>(rt, ma, mw, p);
        return launch_gemm_pair<128>(rt, ma, mw, p);
    }
    if (bn == 256) return launch_gemm<256>(rt, ma, mw, p);
    if (bn == 192) return launch_gemm<192>(rt, ma, mw, p);
    return launch_gemm<128>(rt, ma, mw, p);
}

/// Upper bound of the built-in scratch: enough for m * K_aug f16 activations plus
/// m row scales, e.g. 963 rows at K = 4096, G = 64, or 3847 rows at K = 1024.
constexpr size_t kStaticScratchBytes = size_t(8) << 20;

/// The scratch itself lives in the library image: every GPU that loads the
/// library holds these 8 MiB until the process exits. In host code this name is
/// only a stand-in; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void *g_static_scratch_addr[kMaxDevices] = {};

/// Device address of the built-in scratch on the runtime's device (which the
/// caller has made current). Looked up once per device, on the first call.
Result static_scratch_address(TesslRuntime *rt, void **out)
{
    if (rt->device < 0 || rt->device >= kMaxDevices)
        return fmt("gemm_q4_mlx_tensorops_noalloc: device ordinal %d is outside 0..%d", rt->device, kMaxDevices - 1);
    if (!g_static_scratch_addr[rt->device]) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            cudaGetLastError();
            return fmt("gemm_q4_mlx_tensorops_noalloc: cannot resolve the built-in scratch on device %d (%s)",
                       rt->device, cudaGetErrorString(e));
        }
        g_static_scratch_addr[rt->device] = ptr;
    }
    *out = g_static_scratch_addr[rt->device];
    return ok();
}

}  // namespace

namespace nn {

uint32_t gemm_q4_mlx_tensorops_max_k(uint32_t m, uint32_t n, uint32_t group_size)
{
    const uint64_t widest = std::max<uint64_t>(std::max(m, n), 1);
    const uint64_t k = std::min<uint64_t>(0x7fffffffull / widest, 0xffffffffull);
    const uint64_t g = std::max<uint32_t>(group_size, 1);
    return (uint32_t)(k / g * g);
}

Result gemm_q4_mlx_tensorops(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                             const TesslQuantShape &shape, uint32_t m, OutKind out)
{
    PrefillPlan pl{};
    bool empty = false;
    TESSL_TRY(prefill_validate(bank, x_bf16, y, shape, m, out, &pl, &empty));
    if (empty) return ok();
    rt->prefill_last_bn = 0, rt->prefill_last_pair = 0;
    if (rt->prefill_force_bn == 0 && rt->prefill_force_pair < 0) {
        bool handled = false;  // a few rows: batches of 8 on the tensor-core GEMV kernel
        TESSL_TRY(prefill_as_small_batches(rt, bank, x_bf16, y, shape, m, out, &handled));
        if (handled) return ok();
    }
    // Scratch: the augmented f16 activations [m, k_aug] and the row scales [m].
    void *scratch = nullptr;
    TESSL_TRY(scratch_reserve(rt, pl.need, &scratch));
    return prefill_launch(rt, bank, x_bf16, y, m, out, pl, scratch);
}

/// `gemm_q4_mlx_tensorops` for callers that must not allocate device memory
/// while they run: serving loops that forbid anything that can synchronise the
/// device or fail for lack of memory in steady state, or code inside another
/// framework's allocator discipline. The regular entry grows a scratch buffer
/// with cudaMalloc whenever a call needs more than any earlier one; this one
/// puts the same intermediate data (the f16 copy of X with its group sums, and
/// the row scales) into a fixed array inside the library and refuses shapes
/// that do not fit. Same validation, same kernels, same bits.
///
/// The first call on a device resolves the array's address (no allocation, but
/// a synchronous query of the CUDA runtime). The array is shared by
/// every call and every runtime on that device and keeps the last call's
/// contents; the pre-pass rewrites every byte a call later reads, so nothing has
/// to start at zero, but two calls that overlap on the GPU (two streams, two
/// runtimes) race on it and must be serialised by the caller.
Result gemm_q4_mlx_tensorops_noalloc(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16,
                                     const TesslBuf &y, const TesslQuantShape &shape, uint32_t m, OutKind out)
{
    PrefillPlan pl{};
    bool empty = false;
    TESSL_TRY(prefill_validate(bank, x_bf16, y, shape, m, out, &pl, &empty));
    if (empty) return ok();
    rt->prefill_last_bn = 0, rt->prefill_last_pair = 0;
    if (rt->prefill_force_bn == 0 && rt->prefill_force_pair < 0) {
        bool handled = false;  // needs no scratch at all
        TESSL_TRY(prefill_as_small_batches(rt, bank, x_bf16, y, shape, m, out, &handled));
        if (handled) return ok();
    }
    if (pl.need > kStaticScratchBytes) {
        return fmt("gemm_q4_mlx_tensorops_noalloc: m = %u rows of %u columns need %zu bytes of scratch but the "
                   "built-in scratch holds %zu; use gemm_q4_mlx_tensorops, which allocates",
                   m, pl.k, pl.need, kStaticScratchBytes);
    }
    void *scratch = nullptr;
    TESSL_TRY(static_scratch_address(rt, &scratch));
    return prefill_launch(rt, bank, x_bf16, y, m, out, pl, scratch);
}

}  // namespace nn
}  // namespace tessl
