// 8-bit affine GEMV kernels for sm_100a.
//
//  * gemv_q8: the reference's Q8 convention (`nn::gemv_q8`, src/nn.rs:716-795;
//    kernels/gemv_q8.metal in the reference project): signed int8 codes,
//    f32 scale and zero per group, w = scale * (q - zero), f32 x, M = 1.
//  * gemm_q8_mlx: MLX's bank convention at eight bits: unsigned codes, one
//    bf16 (scale, bias) pair per group, w = scale * code + bias, bf16 x, M <= 8.
//
// Same shape as the Q4 kernels: a block owns R rows, its warps split K into
// 512-column chunks, a lane reads 16 codes per row and chunk with one 128-bit
// load and all R loads are issued before any is used. Codes become floats by a
// byte permute into the mantissa of 2^23 and one subtraction (exact).
#include "q4_common.cuh"
#include "runtime.h"

namespace tessl {
namespace {

constexpr int kChunk8 = 512;  // 32 lanes x 16 codes

/// Byte B of `u` (an unsigned code 0..255) as the float 2^23 + code.
template <int B>
__device__ __forceinline__ float byte_to_f2p23(uint32_t u)
{
    return __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7440u | B));
}

/// The 16 unsigned codes of `w` as exact floats.
__device__ __forceinline__ void codes16(const uint4 &w, float (&q)[16])
{
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        q[4 * j + 0] = byte_to_f2p23<0>(words[j]) - 8388608.0f;
        q[4 * j + 1] = byte_to_f2p23<1>(words[j]) - 8388608.0f;
        q[4 * j + 2] = byte_to_f2p23<2>(words[j]) - 8388608.0f;
        q[4 * j + 3] = byte_to_f2p23<3>(words[j]) - 8388608.0f;
    }
}

struct Q8Params {
    const uint8_t *codes;
    const uint32_t *sb;     // mlx: bf16 (scale, bias) pairs
    const float *scales;    // i8: f32 tables
    const float *zeros;
    const void *x;
    void *y;
    uint32_t rows, cols, group_size;
    int out_bf16;
};

/// MLX-layout Q8, M activation rows, R output rows per block.
template <int M, int R>
__global__ void __launch_bounds__(128) q8_mlx_kernel(const Q8Params p)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const uint32_t rows = p.rows, cols = p.cols;
    const uint32_t row0 = blockIdx.x * R;
    const uint32_t gpr = cols / p.group_size;
    const uint16_t *x = static_cast<const uint16_t *>(p.x);
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

    for (uint32_t k0 = warp * kChunk8 + lane * 16; k0 < cols; k0 += nwarps * kChunk8) {
        uint4 wq[R];
        uint32_t sbw[R];
        const uint32_t g = k0 / p.group_size;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t row = min(row0 + r, rows - 1);
            wq[r] = dev::ldg_stream16(p.codes + (size_t)row * cols + k0);
            sbw[r] = dev::ldg_stream4(p.sb + (size_t)row * gpr + g);
        }
        float xs[M][16];
        float xsum[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 *xp = reinterpret_cast<const uint4 *>(x + (size_t)m * cols + k0);
            float t = 0.0f;
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const uint4 xv = __ldg(xp + v);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    xs[m][8 * v + 2 * j] = dev::bf16_lo(xw[j]);
                    xs[m][8 * v + 2 * j + 1] = dev::bf16_hi(xw[j]);
                    t += xs[m][8 * v + 2 * j] + xs[m][8 * v + 2 * j + 1];
                }
            }
            xsum[m] = t;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float q[16];
            codes16(wq[r], q);
            const float scale = dev::bf16_lo(sbw[r]), bias = dev::bf16_hi(sbw[r]);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    d0 = fmaf(xs[m][i], q[i], d0);
                    d1 = fmaf(xs[m][i + 1], q[i + 1], d1);
                }
                acc[r][m] = fmaf(scale, d0 + d1, fmaf(bias, xsum[m], acc[r][m]));
            }
        }
    }

    __shared__ float red[4][R * M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float v = dev::warp_sum(acc[r][m]);
            if (lane == 0) red[warp][r * M + m] = v;
        }
    __syncthreads();
    const int t = threadIdx.x;
    if (t < R * M) {
        const int r = t / M, m = t % M;
        const uint32_t row = row0 + r;
        if (row < rows) {
            float v = red[0][t];
            for (int w = 1; w < nwarps; ++w) v += red[w][t];
            const size_t idx = (size_t)m * rows + row;
            if (p.out_bf16) {
                static_cast<uint16_t *>(p.y)[idx] = dev::f32_to_bf16_store(v);
            } else {
                static_cast<float *>(p.y)[idx] = v;
            }
        }
    }
}

/// Reference-convention Q8 (int8, f32 scale/zero, f32 x), vector path: needs
/// group_size and cols multiples of 16 so a lane's 16 codes share one group.
template <int R>
__global__ void __launch_bounds__(128) q8_i8_kernel(const Q8Params p)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const uint32_t rows = p.rows, cols = p.cols;
    const uint32_t row0 = blockIdx.x * R;
    const uint32_t gpr = cols / p.group_size;
    const float *x = static_cast<const float *>(p.x);
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    for (uint32_t k0 = warp * kChunk8 + lane * 16; k0 < cols; k0 += nwarps * kChunk8) {
        uint4 wq[R];
        float sc[R], zp[R];
        const uint32_t g = k0 / p.group_size;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t row = min(row0 + r, rows - 1);
            wq[r] = dev::ldg_stream16(p.codes + (size_t)row * cols + k0);
            sc[r] = __ldg(p.scales + (size_t)row * gpr + g);
            zp[r] = __ldg(p.zeros + (size_t)row * gpr + g);
        }
        float xs[16];
        float xsum = 0.0f;
        const float4 *xp = reinterpret_cast<const float4 *>(x + k0);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const float4 xv = __ldg(xp + v);
            xs[4 * v] = xv.x, xs[4 * v + 1] = xv.y, xs[4 * v + 2] = xv.z, xs[4 * v + 3] = xv.w;
            xsum += (xv.x + xv.y) + (xv.z + xv.w);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            // Signed codes: flipping the top bit of each byte gives code + 128 unsigned.
            uint4 u = wq[r];
            u.x ^= 0x80808080u, u.y ^= 0x80808080u, u.z ^= 0x80808080u, u.w ^= 0x80808080u;
            float q[16];
            codes16(u, q);
            float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                d0 = fmaf(xs[i], q[i], d0);
                d1 = fmaf(xs[i + 1], q[i + 1], d1);
            }
            // sum x * (q + 128 - 128 - zero) = dot - (128 + zero) * xsum
            const float dot = fmaf(-(128.0f + zp[r]), xsum, d0 + d1);
            acc[r] = fmaf(sc[r], dot, acc[r]);
        }
    }
    __shared__ float red[4][R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float v = dev::warp_sum(acc[r]);
        if (lane == 0) red[warp][r] = v;
    }
    __syncthreads();
    const int t = threadIdx.x;
    if (t < R && row0 + t < rows) {
        float v = red[0][t];
        for (int w = 1; w < nwarps; ++w) v += red[w][t];
        static_cast<float *>(p.y)[row0 + t] = v;
    }
}

/// Any group size and alignment: one warp per row, lanes stride the columns,
/// w = scale * (q - zero) per element as the reference's scalar path does
/// (kernels/gemv_q8.metal:101-113).
__global__ void __launch_bounds__(128) q8_i8_scalar_kernel(const Q8Params p)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= p.rows) return;
    const uint32_t cols = p.cols, gpr = cols / p.group_size;
    const int8_t *q = reinterpret_cast<const int8_t *>(p.codes) + (size_t)row * cols;
    const float *x = static_cast<const float *>(p.x);
    float acc = 0.0f;
    for (uint32_t c = lane; c < cols; c += 32) {
        const size_t gi = (size_t)row * gpr + c / p.group_size;
        const float w = p.scales[gi] * ((float)q[c] - p.zeros[gi]);
        acc = fmaf(w, x[c], acc);
    }
    acc = dev::warp_sum(acc);
    if (lane == 0) static_cast<float *>(p.y)[row] = acc;
}

template <int M, int R>
Result launch_mlx(TesslRuntime *rt, const Q8Params &p, int warps)
{
    q8_mlx_kernel<M, R><<<(p.rows + R - 1) / R, warps * 32, 0, rt->stream>>>(p);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "q8_mlx launch");
}

}  // namespace

namespace nn {

Result gemv_q8(TesslRuntime *rt, const TesslBuf &packed, const TesslBuf &scales, const TesslBuf &zeros,
               const TesslBuf &x, const TesslBuf &y, uint32_t rows, uint32_t cols, uint32_t group_size)
{
    if (group_size == 0) return "gemv_q8: group_size must be non-zero";
    if (cols % group_size != 0) {
        return fmt("gemv_q8: cols %u is not a multiple of group_size %u; the kernel would silently drop the ragged "
                   "tail group",
                   cols, group_size);
    }
    const uint64_t weights = elems(rows, cols);
    const uint64_t groups = elems(rows, cols / group_size);
    TESSL_TRY(require(packed, weights, 1, "gemv_q8 packed"));
    TESSL_TRY(require(scales, groups, 4, "gemv_q8 scales"));
    TESSL_TRY(require(zeros, groups, 4, "gemv_q8 zeros"));
    TESSL_TRY(require(x, cols, 4, "gemv_q8 x"));
    TESSL_TRY(require(y, rows, 4, "gemv_q8 y"));
    if (rows == 0) return ok();
    const Named writes[] = {{"y", &y}};
    const Named reads[] = {{"packed", &packed}, {"scales", &scales}, {"zeros", &zeros}, {"x", &x}};
    TESSL_TRY(require_disjoint_writes("gemv_q8", writes, 1, reads, 4));
    Q8Params p{};
    p.codes = static_cast<const uint8_t *>(packed.ptr);
    p.scales = static_cast<const float *>(scales.ptr);
    p.zeros = static_cast<const float *>(zeros.ptr);
    p.x = x.ptr;
    p.y = y.ptr;
    p.rows = rows, p.cols = cols, p.group_size = group_size;
    const bool vec = group_size % 16 == 0 && cols % 16 == 0 && ((uintptr_t)packed.ptr & 15u) == 0 &&
                     ((uintptr_t)x.ptr & 15u) == 0 && cols > 0;
    if (vec) {
        const int warps = (int)std::max<uint32_t>(1u, std::min<uint32_t>(4u, (cols + kChunk8 - 1) / kChunk8));
        if ((uint64_t)rows >= (uint64_t)(8 * 3 * rt->sm_count)) {
            q8_i8_kernel<8><<<(rows + 7) / 8, warps * 32, 0, rt->stream>>>(p);
        } else {
            q8_i8_kernel<2><<<(rows + 1) / 2, warps * 32, 0, rt->stream>>>(p);
        }
    } else {
        q8_i8_scalar_kernel<<<(rows + 3) / 4, 128, 0, rt->stream>>>(p);
    }
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "gemv_q8 launch");
}

Result gemm_q8_mlx(TesslRuntime *rt, const TesslBuf &codes, const TesslBuf &sb, const TesslBuf &x_bf16,
                   const TesslBuf &y, const TesslQuantShape &shape, uint32_t m, OutKind out)
{
    const char *entry = "gemm_q8_mlx";
    if (m == 0) return ok();
    if (m > TESSL_GEMM_Q4_MLX_MAX_M) return fmt("%s: M = %u exceeds the small-batch limit %u", entry, m, 8u);
    TESSL_TRY(quant_shape_validate(shape, entry));
    if (shape.group_size % 32 != 0 || 512 % shape.group_size != 0) {
        return fmt("%s: group_size %u is outside the MLX kernel domain {32, 64, 128, 256, 512}", entry,
                   shape.group_size);
    }
    TESSL_TRY(require(codes, elems(shape.rows, shape.cols), 1, std::string(entry) + " codes"));
    TESSL_TRY(require(sb, elems(shape.rows, shape.cols / shape.group_size), 4,
                      std::string(entry) + " scales_biases (bfloat2 per group)"));
    TESSL_TRY(require(x_bf16, elems(m, shape.cols), 2, std::string(entry) + " x_bf16"));
    TESSL_TRY(require(y, elems(m, shape.rows), out == OUT_BF16 ? 2 : 4, std::string(entry) + " y"));
    if (shape.rows == 0) return ok();
    const Named writes[] = {{"y", &y}};
    const Named reads[] = {{"codes", &codes}, {"scales_biases", &sb}, {"x_bf16", &x_bf16}};
    TESSL_TRY(require_disjoint_writes(entry, writes, 1, reads, 3));
    TESSL_TRY(require_aligned16(codes, std::string(entry) + " codes"));
    TESSL_TRY(require_aligned16(x_bf16, std::string(entry) + " x_bf16"));
    {
        // rows of 512 .. 4096 codes in groups of 32 or 64: the tensor-core GEMV kernel (q4_gemv_mma.cuh)
        bool handled = false;
        TESSL_TRY(q8_mlx_mma(rt, codes, sb, x_bf16, y, shape.rows, shape.cols, shape.group_size, m, out, &handled));
        if (handled) return ok();
    }
    Q8Params p{};
    p.codes = static_cast<const uint8_t *>(codes.ptr);
    p.sb = static_cast<const uint32_t *>(sb.ptr);
    p.x = x_bf16.ptr;
    p.y = y.ptr;
    p.rows = shape.rows, p.cols = shape.cols, p.group_size = shape.group_size;
    p.out_bf16 = out == OUT_BF16;
    const int warps = (int)std::max<uint32_t>(1u, std::min<uint32_t>(4u, (shape.cols + kChunk8 - 1) / kChunk8));
    const bool big = (uint64_t)shape.rows >= (uint64_t)(8 * 3 * rt->sm_count);
    switch (m) {
    case 1: return big ? launch_mlx<1, 8>(rt, p, warps) : launch_mlx<1, 2>(rt, p, warps);
    case 2: return big ? launch_mlx<2, 8>(rt, p, warps) : launch_mlx<2, 2>(rt, p, warps);
    case 3: return launch_mlx<3, 4>(rt, p, warps);
    case 4: return launch_mlx<4, 4>(rt, p, warps);
    case 5: return launch_mlx<5, 2>(rt, p, warps);
    case 6: return launch_mlx<6, 2>(rt, p, warps);
    case 7: return launch_mlx<7, 2>(rt, p, warps);
    default: return launch_mlx<8, 2>(rt, p, warps);
    }
}

}  // namespace nn
}  // namespace tessl
