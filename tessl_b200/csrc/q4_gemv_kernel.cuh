// The MLX affine Q4 GEMV / small-batch GEMM kernel for sm_100a.
//
// y[m, row] = sum_k x[m, k] * (scale[row, k/G] * q[row, k] + bias[row, k/G])
//
// The work is a one-pass stream of the packed weights, so the kernel is built
// around bytes in flight and instructions per byte:
//
//   * Persistent blocks. The grid is a few blocks per SM; block b walks the row
//     groups b, b + gridDim, ... so every SM streams the same number of bytes to
//     within one small group, whatever the row count.
//   * Split K across the warps of a block. Warp w owns the 1024-column chunks
//     w, w + W, ... of every row (NCH chunks, a compile-time count), so the block
//     as a whole reads complete, contiguous packed rows, and a warp's slice of x
//     (32 bf16 per lane and chunk) is loaded ONCE per launch and stays packed
//     in registers.
//   * A lane reads 16 bytes (32 nibbles, never more than one quantization
//     group) per row and chunk with a non-allocating 128-bit load. The loads of
//     the next row group are issued before the current one is computed.
//   * No integer-to-float conversion and no activation unpacking: one LOP3
//     turns two nibbles of a word into two bf16 values 128 + q (nibble in the
//     mantissa of 0x4300), and the Blackwell mixed-precision FMA
//     (fma.rn.f32.bf16: bf16 * bf16 + f32, exact product) multiplies them with
//     the packed bf16 activations straight into an f32 accumulator. That is
//     7 ALU + 8 FMA instructions per 8 weights. The 128 * sum(x) excess is
//     removed once per 32 weights.
//   * Per lane the group's affine is scale * dot + bias * sum(x) in f32 (the
//     reference's `qdot16`, kernels/q4_mlx_dot.h:72-94 of the reference
//     project); lanes are combined by a transposing shuffle reduction, warps
//     through double-buffered shared memory in a fixed order.
//
// A row's summation order depends only on `cols`, never on which bank, launch or
// epilogue it belongs to, so fused gate/up, K/V and Q/K/V launches are
// bit-identical to separate launches (kernels/gemv_q4_mlx.metal:634-655 of the
// reference project makes the same promise).
#pragma once

#include "q4_common.cuh"

namespace tessl {
namespace q4k {

enum : int { EPI_STORE = 0, EPI_ADD_RESID = 1, EPI_GATE_UP_GELU = 2, EPI_GATE_UP_SILU = 3 };

struct Seg {
    const uint8_t *packed0;
    const uint32_t *sb0;
    const uint8_t *packed1;  // second bank of a gate/up launch
    const uint32_t *sb1;
    void *out;
    const float *resid;
    uint32_t rows;
    uint32_t group_begin;  // first row group of this bank within the launch
};

struct Params {
    Seg seg[3];
    int nseg;
    uint32_t ngroups;   // row groups over all banks
    const uint16_t *x;  // bf16 [m, cols]
    uint32_t cols;
    uint32_t group_shift;  // log2(group_size)
    int epi;
    int out_bf16;
    // Host side only: the TesslPeerGather of a column-sharded launch whose kernel exchanges its own
    // outputs (q4_gemv_mma.cuh), else null. Kernels other than that one never read it.
    const void *peer;
    int peer_defer;     // with `peer`: tell the peers, do not wait for them (the reader of the gathered vector does)
    const void *xwait;  // a TesslPeerGather whose buffer is x and whose last exchange was deferred, else null
    // Host side only: the banks are in the staged layout (units of 8 rows in the tensor-core kernel's
    // shared-memory form); only that kernel takes them.
    int staged;
};

constexpr int kChunk = 1024;  // columns one warp covers per step: 32 lanes x 32 nibbles
constexpr uint32_t kMagic = 0x43004300u;  // two bf16 128.0

/// acc += bf16(half H of a) * bf16(half H' of b), product exact, one FMA-pipe instruction.
#define TESSL_MIXED_FMA(acc, qreg, QH, xreg, XH)                                                     \
    asm("{\n\t.reg .b16 ql, qh, xl, xh;\n\tmov.b32 {ql, qh}, %1;\n\tmov.b32 {xl, xh}, %2;\n\t"       \
        "fma.rn.f32.bf16 %0, " QH ", " XH ", %0;\n\t}"                                               \
        : "+f"(acc)                                                                                  \
        : "r"(qreg), "r"(xreg))

/// (a & mask) | orv as ONE LOP3. Written as inline PTX because the compiler
/// otherwise emits a separate AND and OR here (measured: 32 LOP3 per 32
/// weights instead of 16).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t orv)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}

/// sum over the 32 nibbles of `w` of x_k * (128 + q_k); `xr` holds the lane's 32
/// activations as 16 packed bf16 pairs (x[2t], x[2t+1]).
__device__ __forceinline__ float dot32_biased(const uint4 &w, const uint32_t (&xr)[16])
{
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t w0 = words[j];
        // nibble pairs (i, i + 4) as two bf16 values 128 + q
        const uint32_t q04 = and_or(w0, 0x000f000fu, kMagic);
        const uint32_t q15 = and_or(w0 >> 4, 0x000f000fu, kMagic);
        const uint32_t q26 = and_or(w0 >> 8, 0x000f000fu, kMagic);
        const uint32_t q37 = and_or(w0 >> 12, 0x000f000fu, kMagic);
        TESSL_MIXED_FMA(d0, q04, "ql", xr[4 * j + 0], "xl");  // k = 8j + 0
        TESSL_MIXED_FMA(d1, q15, "ql", xr[4 * j + 0], "xh");  // 8j + 1
        TESSL_MIXED_FMA(d0, q26, "ql", xr[4 * j + 1], "xl");  // 8j + 2
        TESSL_MIXED_FMA(d1, q37, "ql", xr[4 * j + 1], "xh");  // 8j + 3
        TESSL_MIXED_FMA(d0, q04, "qh", xr[4 * j + 2], "xl");  // 8j + 4
        TESSL_MIXED_FMA(d1, q15, "qh", xr[4 * j + 2], "xh");  // 8j + 5
        TESSL_MIXED_FMA(d0, q26, "qh", xr[4 * j + 3], "xl");  // 8j + 6
        TESSL_MIXED_FMA(d1, q37, "qh", xr[4 * j + 3], "xh");  // 8j + 7
    }
    return d0 + d1;
}

/// Sum of the lane's 32 activations in f32.
__device__ __forceinline__ float xsum32(const uint32_t (&xr)[16])
{
    float p[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int t = 0; t < 16; ++t) p[t & 3] += dev::bf16_lo(xr[t]) + dev::bf16_hi(xr[t]);
    return (p[0] + p[1]) + (p[2] + p[3]);
}

/// Loads the lane's 32 activations of row m at column k0 (or zeros past the end).
__device__ __forceinline__ void load_x32(const uint16_t *x, size_t off, bool live, uint32_t (&xr)[16])
{
    const uint4 *xp = reinterpret_cast<const uint4 *>(x + off);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        const uint4 xv = live ? __ldg(xp + v) : make_uint4(0, 0, 0, 0);
        xr[4 * v] = xv.x, xr[4 * v + 1] = xv.y, xr[4 * v + 2] = xv.z, xr[4 * v + 3] = xv.w;
    }
}

/// Reduces V per-lane values over the warp with V - 1 + log2(32 / V) shuffles:
/// afterwards the lanes with (lane & (32 / V - 1)) == 0 hold, in v[0], the warp
/// total of value `owned_index(lane)`.
template <int V>
__device__ __forceinline__ void transpose_reduce(float (&v)[V], int lane)
{
    static_assert(V == 1 || V == 2 || V == 4 || V == 8 || V == 16 || V == 32, "V must be a power of two");
    int off = 16;
#pragma unroll
    for (int s = V / 2; s >= 1; s >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < s; ++i) {
            const float send = upper ? v[i] : v[i + s];
            const float keep = upper ? v[i + s] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
        off >>= 1;
    }
    for (; off >= 1; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}

template <int V>
__device__ __forceinline__ int owned_index(int lane)
{
    int idx = 0, off = 16;
#pragma unroll
    for (int s = V / 2; s >= 1; s >>= 1) {
        if (lane & off) idx += s;
        off >>= 1;
    }
    return idx;
}

}  // namespace q4k
}  // namespace tessl
