// MLX affine Q4 GEMV (M = 1) and small-batch GEMM (M <= 8) for sm_100a, with the
// host-side wrappers that mirror the reference's `nn::gemv_q4_mlx_*` and
// `nn::gemm_q4_mlx` (src/nn.rs:3982-4619 of the reference project).
//
// The work is a memory-bound stream of the packed weights, so the kernel is
// organised around bytes in flight, not arithmetic:
//
//   * a block owns R consecutive output rows of one bank and its warps split K
//     into 1024-column chunks (warp w takes chunks w, w + W, ...), so the block
//     as a whole reads R complete, contiguous packed rows;
//   * a lane reads 16 bytes (32 nibbles, at most one quantization group) per
//     row and chunk with a non-allocating 128-bit load, and issues the loads of
//     all R rows before it touches any of them;
//   * the lane's 32 activations are widened to f32 registers once per chunk and
//     reused by all R rows;
//   * nibbles become floats without an integer-to-float conversion: a byte
//     permute drops each one into the mantissa of 128.0f, the dot product runs
//     on 128 + q, and the 128 * sum(x) excess is removed once per 32 weights;
//   * per lane the group's affine is applied as scale * dot + bias * sum(x) in
//     f32 (the reference's `qdot16`, kernels/q4_mlx_dot.h:72-94), lanes are
//     combined by shuffles, warps through shared memory in a fixed order.
//
// A row's summation order depends only on `cols`, never on which bank, launch
// or epilogue it belongs to, so the fused gate/up, K/V and Q/K/V launches are
// bit-identical to separate launches, as in the reference
// (kernels/gemv_q4_mlx.metal:634-655).
#include "q4_common.cuh"
#include "runtime.h"

namespace tessl {
namespace {

enum : int { EPI_STORE = 0, EPI_ADD_RESID = 1, EPI_GATE_UP_GELU = 2, EPI_GATE_UP_SILU = 3 };

struct Q4Seg {
    const uint8_t *packed0;
    const uint32_t *sb0;
    const uint8_t *packed1;  // second bank of a gate/up launch
    const uint32_t *sb1;
    void *out;
    const float *resid;
    uint32_t rows;
    uint32_t block_begin;  // first block of this bank within the grid
};

struct Q4GemvParams {
    Q4Seg seg[3];
    int nseg;
    const uint16_t *x;  // bf16 [m, cols]
    uint32_t cols;
    uint32_t group_shift;  // log2(group_size)
    int epi;
    int out_bf16;
};

constexpr int kChunk = 1024;  // columns one warp covers per step: 32 lanes x 32 nibbles

/// sum_i xs[i] * (128 + q_i) over the 32 nibbles of `w`, two chains.
__device__ __forceinline__ float dot32_biased(const uint4 &w, const float (&xs)[32])
{
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t lo = words[j] & 0x0f0f0f0fu;         // nibbles 0, 2, 4, 6
        const uint32_t hi = (words[j] >> 4) & 0x0f0f0f0fu;  // nibbles 1, 3, 5, 7
        d0 = fmaf(xs[8 * j + 0], dev::nib_byte_to_f128<0>(lo), d0);
        d1 = fmaf(xs[8 * j + 1], dev::nib_byte_to_f128<0>(hi), d1);
        d0 = fmaf(xs[8 * j + 2], dev::nib_byte_to_f128<1>(lo), d0);
        d1 = fmaf(xs[8 * j + 3], dev::nib_byte_to_f128<1>(hi), d1);
        d0 = fmaf(xs[8 * j + 4], dev::nib_byte_to_f128<2>(lo), d0);
        d1 = fmaf(xs[8 * j + 5], dev::nib_byte_to_f128<2>(hi), d1);
        d0 = fmaf(xs[8 * j + 6], dev::nib_byte_to_f128<3>(lo), d0);
        d1 = fmaf(xs[8 * j + 7], dev::nib_byte_to_f128<3>(hi), d1);
    }
    return d0 + d1;
}

/// The 32 nibbles of `w` as floats 128 + q.
__device__ __forceinline__ void dequant32_biased(const uint4 &w, float (&qf)[32])
{
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t lo = words[j] & 0x0f0f0f0fu;
        const uint32_t hi = (words[j] >> 4) & 0x0f0f0f0fu;
        qf[8 * j + 0] = dev::nib_byte_to_f128<0>(lo);
        qf[8 * j + 1] = dev::nib_byte_to_f128<0>(hi);
        qf[8 * j + 2] = dev::nib_byte_to_f128<1>(lo);
        qf[8 * j + 3] = dev::nib_byte_to_f128<1>(hi);
        qf[8 * j + 4] = dev::nib_byte_to_f128<2>(lo);
        qf[8 * j + 5] = dev::nib_byte_to_f128<2>(hi);
        qf[8 * j + 6] = dev::nib_byte_to_f128<3>(lo);
        qf[8 * j + 7] = dev::nib_byte_to_f128<3>(hi);
    }
}

/// M activation rows, NB banks (2 for gate/up), R output rows per block.
template <int M, int NB, int R>
__global__ void __launch_bounds__(128) q4_gemv_kernel(const Q4GemvParams p)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    int s = 0;
    if (p.nseg > 1 && blockIdx.x >= p.seg[1].block_begin) s = 1;
    if (p.nseg > 2 && blockIdx.x >= p.seg[2].block_begin) s = 2;
    const Q4Seg sg = p.seg[s];
    const uint32_t rows = sg.rows, cols = p.cols;
    const uint32_t row0 = (blockIdx.x - sg.block_begin) * R;
    const uint32_t gpr = cols >> p.group_shift;
    const size_t row_bytes = cols >> 1;
    const uint8_t *packed[2] = {sg.packed0, sg.packed1};
    const uint32_t *sbp[2] = {sg.sb0, sg.sb1};

    float acc[R][NB][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][b][m] = 0.0f;

    for (uint32_t k0 = warp * kChunk + lane * 32; k0 < cols; k0 += nwarps * kChunk) {
        // Every row's weights first: R * NB independent 16-byte loads in flight.
        uint4 wq[R][NB];
        uint32_t sbw[R][NB];
        const uint32_t g = k0 >> p.group_shift;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            // Rows past the bank's end re-read its last row; their sums are never stored.
            const uint32_t row = min(row0 + r, rows - 1);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                wq[r][b] = dev::ldg_stream16(packed[b] + row * row_bytes + (k0 >> 1));
                sbw[r][b] = dev::ldg_stream4(sbp[b] + (size_t)row * gpr + g);
            }
        }
        if constexpr (M == 1) {
            float xs[32];
            const uint4 *xp = reinterpret_cast<const uint4 *>(p.x + k0);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 xv = __ldg(xp + v);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    xs[8 * v + 2 * j] = dev::bf16_lo(xw[j]);
                    xs[8 * v + 2 * j + 1] = dev::bf16_hi(xw[j]);
                }
            }
            float part[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) part[i] = (xs[4 * i] + xs[4 * i + 1]) + (xs[4 * i + 2] + xs[4 * i + 3]);
            const float xsum = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const float dot = fmaf(-128.0f, xsum, dot32_biased(wq[r][b], xs));
                    const float scale = dev::bf16_lo(sbw[r][b]), bias = dev::bf16_hi(sbw[r][b]);
                    acc[r][b][0] = fmaf(scale, dot, fmaf(bias, xsum, acc[r][b][0]));
                }
            }
        } else {
            // Small batch: the weights of a row are expanded once and every
            // activation row is run against them; x stays packed and is widened
            // as it is used.
            uint4 xq[M][4];
            float xsum[M];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(p.x + (size_t)m * cols + k0);
                float t = 0.0f;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    xq[m][v] = __ldg(xp + v);
                    const uint32_t xw[4] = {xq[m][v].x, xq[m][v].y, xq[m][v].z, xq[m][v].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) t += dev::bf16_lo(xw[j]) + dev::bf16_hi(xw[j]);
                }
                xsum[m] = t;
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float qf[32];
                dequant32_biased(wq[r][0], qf);
                const float scale = dev::bf16_lo(sbw[r][0]), bias = dev::bf16_hi(sbw[r][0]);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const uint32_t xw[4] = {xq[m][v].x, xq[m][v].y, xq[m][v].z, xq[m][v].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            d0 = fmaf(dev::bf16_lo(xw[j]), qf[8 * v + 2 * j], d0);
                            d1 = fmaf(dev::bf16_hi(xw[j]), qf[8 * v + 2 * j + 1], d1);
                        }
                    }
                    const float dot = fmaf(-128.0f, xsum[m], d0 + d1);
                    acc[r][0][m] = fmaf(scale, dot, fmaf(bias, xsum[m], acc[r][0][m]));
                }
            }
        }
    }

    // Lanes, then warps (fixed order), then the epilogue: one thread per output.
    __shared__ float red[4][R * NB * M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float v = dev::warp_sum(acc[r][b][m]);
                if (lane == 0) red[warp][(r * NB + b) * M + m] = v;
            }
    __syncthreads();
    const int t = threadIdx.x;
    if (t < R * M) {
        const int r = t / M, m = t % M;
        const uint32_t row = row0 + r;
        if (row < rows) {
            float sum[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float v = red[0][(r * NB + b) * M + m];
                for (int w = 1; w < nwarps; ++w) v += red[w][(r * NB + b) * M + m];
                sum[b] = v;
            }
            const size_t idx = (size_t)m * rows + row;
            float v = sum[0];
            if (p.epi == EPI_ADD_RESID) {
                v = v + sg.resid[idx];
            } else if (p.epi == EPI_GATE_UP_SILU) {
                v = dev::silu(sum[0]) * sum[NB - 1];
            } else if (p.epi == EPI_GATE_UP_GELU) {
                v = dev::gelu_pytorch_tanh(sum[0]) * sum[NB - 1];
            }
            if (p.out_bf16) {
                static_cast<uint16_t *>(sg.out)[idx] = dev::f32_to_bf16_store(v);
            } else {
                static_cast<float *>(sg.out)[idx] = v;
            }
        }
    }
}

__global__ void swiglu_kernel(const float *gate, const float *up, void *out, uint32_t n, int out_bf16)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = dev::silu(gate[i]) * up[i];
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

uint32_t log2_u32(uint32_t v)
{
    uint32_t s = 0;
    while ((1u << s) < v) ++s;
    return s;
}

template <int M, int NB, int R>
Result launch_one(TesslRuntime *rt, const Q4GemvParams &p, uint32_t blocks, int warps)
{
    q4_gemv_kernel<M, NB, R><<<blocks, warps * 32, 0, rt->stream>>>(p);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "q4_gemv launch");
}

/// Rows per block: as many as keep the grid at a few blocks per SM.
int pick_rows_per_block(const TesslRuntime *rt, uint64_t total_rows, int max_r)
{
    int r = max_r;
    while (r > 2 && (total_rows + r - 1) / r < (uint64_t)(3 * rt->sm_count)) r >>= 1;
    return r;
}

/// Fills block_begin for each segment and launches the right instantiation.
Result launch_q4_gemv(TesslRuntime *rt, Q4GemvParams p, int m, int nb)
{
    uint64_t total_rows = 0;
    for (int s = 0; s < p.nseg; ++s) total_rows += p.seg[s].rows;
    const int warps = (int)std::min<uint32_t>(4u, (p.cols + kChunk - 1) / kChunk);
    const int max_r = (m == 1 && nb == 1) ? 16 : (m == 1 ? 8 : (m <= 2 ? 8 : (m <= 4 ? 4 : 2)));
    const int r = pick_rows_per_block(rt, total_rows, max_r);
    uint32_t blocks = 0;
    for (int s = 0; s < p.nseg; ++s) {
        p.seg[s].block_begin = blocks;
        blocks += (p.seg[s].rows + r - 1) / r;
    }
    if (blocks == 0) return ok();
#define TESSL_CASE(MM, NBB, RR) \
    if (m == MM && nb == NBB && r == RR) return launch_one<MM, NBB, RR>(rt, p, blocks, warps)
    TESSL_CASE(1, 1, 16);
    TESSL_CASE(1, 1, 8);
    TESSL_CASE(1, 1, 4);
    TESSL_CASE(1, 1, 2);
    TESSL_CASE(1, 2, 8);
    TESSL_CASE(1, 2, 4);
    TESSL_CASE(1, 2, 2);
    TESSL_CASE(2, 1, 8);
    TESSL_CASE(2, 1, 4);
    TESSL_CASE(2, 1, 2);
    TESSL_CASE(3, 1, 4);
    TESSL_CASE(3, 1, 2);
    TESSL_CASE(4, 1, 4);
    TESSL_CASE(4, 1, 2);
    TESSL_CASE(5, 1, 2);
    TESSL_CASE(6, 1, 2);
    TESSL_CASE(7, 1, 2);
    TESSL_CASE(8, 1, 2);
#undef TESSL_CASE
    return fmt("q4_gemv: no kernel for m=%d banks=%d rows_per_block=%d", m, nb, r);
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

Result check_alignment(const TesslQ4MlxBank &b, const std::string &what)
{
    TESSL_TRY(require_aligned16(b.packed, what + " packed"));
    if (((uintptr_t)b.scales_biases.ptr & 3u) != 0)
        return fmt("%s scales_biases: device pointer must be 4-byte aligned", what.c_str());
    return ok();
}

}  // namespace

namespace nn {

Result gemv_q4_mlx_simd(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                        const TesslQuantShape &shape, uint32_t layout, const TesslBuf *resid, OutKind out)
{
    const char *entry = resid ? "gemv_q4_mlx_simd_add" : "gemv_q4_mlx_simd";
    TESSL_TRY(refuse_layout(layout, entry));
    TESSL_TRY(q4_bank_validate(bank, shape, entry));
    TESSL_TRY(require(x_bf16, shape.cols, 2, std::string(entry) + " x_bf16"));
    TESSL_TRY(require(y, shape.rows, out == OUT_BF16 ? 2 : 4, std::string(entry) + " y"));
    if (resid) TESSL_TRY(require(*resid, shape.rows, 4, std::string(entry) + " resid"));
    if (shape.rows == 0) return ok();
    const Named writes[] = {{"y", &y}};
    const Named reads[] = {{"packed", &bank.packed}, {"scales_biases", &bank.scales_biases}, {"x_bf16", &x_bf16}};
    TESSL_TRY(require_disjoint_writes(entry, writes, 1, reads, 3));
    TESSL_TRY(check_alignment(bank, entry));
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
    return launch_q4_gemv(rt, p, 1, 1);
}

Result gemv_q4_mlx_gate_up(TesslRuntime *rt, const char *entry, const char *what, bool silu,
                           const TesslQ4MlxBank &gate, const TesslQ4MlxBank &up, const TesslBuf &x,
                           const TesslBuf &mid, const TesslQuantShape &shape, uint32_t layout, bool mid_as_bf16)
{
    TESSL_TRY(refuse_layout(layout, entry));
    TESSL_TRY(q4_bank_validate(gate, shape, std::string(entry) + " gate"));
    TESSL_TRY(q4_bank_validate(up, shape, std::string(entry) + " up"));
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
    TESSL_TRY(check_alignment(gate, std::string(entry) + " gate"));
    TESSL_TRY(check_alignment(up, std::string(entry) + " up"));
    TESSL_TRY(require_aligned16(x, std::string(entry) + " x"));
    Q4GemvParams p{};
    p.seg[0] = make_seg(gate, &up, mid, nullptr, shape.rows);
    p.nseg = 1;
    p.x = static_cast<const uint16_t *>(x.ptr);
    p.cols = shape.cols;
    p.group_shift = log2_u32(shape.group_size);
    p.epi = silu ? EPI_GATE_UP_SILU : EPI_GATE_UP_GELU;
    p.out_bf16 = mid_as_bf16;
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
                                                          out_as_bf16 ? 1 : 0);
    rt->dispatch_count += 1;
    return cuda_check(rt, cudaGetLastError(), "swiglu launch");
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
