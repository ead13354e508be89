/* CPU oracle for the MLX affine-quantized matmul path of bharathvbcr/tessl.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the arithmetic the
 * reference's Metal kernels and its own Rust test references perform, so the
 * CUDA kernels can be checked on a machine that cannot run Metal. Nothing in
 * the shipped library links, loads or calls it; only the tests, the smoke
 * check and the CPU-baseline legs of the benchmark do.
 *
 * Two kinds of function live here:
 *
 *  - "semantic" oracles, which follow the reference's *test* references
 *    (f64 accumulation of the dequantized product). They define what the
 *    right answer is.
 *  - "order-faithful" oracles, which follow the reference's *kernels*
 *    statement by statement (per-lane partial sums, the 16^k prescale, the
 *    simdgroup reduction), in f32. They are pinned twice: against the
 *    known-answer words the reference's tests record for every Q4 kernel entry
 *    (tests/q4_kernels_template.rs:436-1494), and - Q8 included, for which the
 *    reference recorded no vectors - bit for bit against the reference's own
 *    kernel sources compiled for the CPU (`_ref/`, built by build.py from
 *    ref_shim/; tests/test_oracle_ref.py).
 *
 * Every function cites the reference file:line it follows, by the file's path
 * inside the reference project.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ RNG --- */

/* splitmix64 as the reference's tests use it: the constructor XORs the seed
 * with the golden-ratio constant and every draw adds that constant before
 * mixing (tests/common/mod.rs:153-166; tests/q4_kernels_template.rs:33-53). */
ORC_API uint64_t orc_splitmix_new(uint64_t seed) { return seed ^ 0x9e3779b97f4a7c15ull; }

ORC_API uint64_t orc_splitmix_next(uint64_t *state)
{
    *state += 0x9e3779b97f4a7c15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

/* Uniform in [-1, 1): the top 24 bits over 2^23, minus one
 * (tests/common/mod.rs:176-179; tests/q4_kernels_template.rs:49-52). */
ORC_API float orc_splitmix_unit(uint64_t *state)
{
    return (float)(orc_splitmix_next(state) >> 40) / 8388608.0f - 1.0f;
}

/* ----------------------------------------------------------------- bf16 --- */

static inline uint32_t f32_bits(float x)
{
    uint32_t b;
    memcpy(&b, &x, 4);
    return b;
}

static inline float bits_f32(uint32_t b)
{
    float x;
    memcpy(&x, &b, 4);
    return x;
}

/* Host f32 -> bf16, round to nearest even, NaN quieted with its sign and top
 * payload kept (src/tensor.rs:804-813). */
ORC_API uint16_t orc_f32_to_bf16_bits(float x)
{
    uint32_t bits = f32_bits(x);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t round = (bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16;
    return (uint16_t)round;
}

/* f32 -> bf16 as a GPU cast stores it: any NaN becomes 0x7fc0 and an f32
 * subnormal flushes to a zero of its sign (src/tensor.rs:815-831). */
ORC_API uint16_t orc_f32_to_bf16_bits_gpu(float x)
{
    uint32_t bits = f32_bits(x);
    uint32_t m = bits & 0x7fffffffu;
    if (m > 0x7f800000u) return 0x7fc0u;
    if (m < 0x00800000u) return (uint16_t)((bits >> 16) & 0x8000u);
    return orc_f32_to_bf16_bits(x);
}

/* src/tensor.rs:833-835. */
ORC_API float orc_bf16_bits_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

ORC_API void orc_f32_to_bf16_array(const float *src, uint16_t *dst, size_t n)
{
    for (size_t i = 0; i < n; ++i) dst[i] = orc_f32_to_bf16_bits(src[i]);
}

/* -------------------------------------------------------- MLX Q4 format --- */

/* Two nibbles per byte, low nibble first (tests/common/mod.rs:516-521), which
 * is the little-endian byte image of MLX's U32 words with element i at bits
 * 4i..4i+4 (tests/qwen35_mlx_q4.rs:100-110; src/qwen35_q4.rs:10-21). */
ORC_API void orc_q4_pack(const uint8_t *nibbles, size_t n, uint8_t *packed)
{
    for (size_t i = 0; i < n; i += 2) {
        uint8_t lo = nibbles[i] & 0x0f;
        uint8_t hi = (i + 1 < n) ? (nibbles[i + 1] & 0x0f) : 0;
        packed[i / 2] = (uint8_t)(lo | (hi << 4));
    }
}

/* Inverse of orc_q4_pack: nibble i of the matrix, unsigned 0..15. */
ORC_API void orc_q4_unpack(const uint8_t *packed, size_t n, uint8_t *nibbles)
{
    for (size_t i = 0; i < n; ++i) nibbles[i] = (uint8_t)((packed[i / 2] >> (4 * (i & 1))) & 0x0f);
}

/* Interleave separate scale and bias arrays into (scale, bias) bf16 pairs,
 * one per group (src/loader.rs:309-314). */
ORC_API void orc_interleave_scales_biases(const uint16_t *scales, const uint16_t *biases, size_t groups,
                                          uint16_t *sb)
{
    for (size_t g = 0; g < groups; ++g) {
        sb[2 * g] = scales[g];
        sb[2 * g + 1] = biases[g];
    }
}

/* Dense f32 image of a bank: w = scale * q + bias with a separate f32 multiply
 * and add, scale and bias read as the bf16 values the kernel loads
 * (tests/common/mod.rs:528-547; tests/qwen35_mlx_q4.rs:87-97). */
ORC_API void orc_q4_dequant(const uint8_t *packed, const uint16_t *sb, size_t rows, size_t cols, size_t group,
                            float *dense)
{
    const size_t gpr = cols / group;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        for (size_t c = 0; c < cols; ++c) {
            const size_t i = (size_t)r * cols + c;
            const size_t gi = (size_t)r * gpr + c / group;
            const float s = orc_bf16_bits_to_f32(sb[2 * gi]);
            const float b = orc_bf16_bits_to_f32(sb[2 * gi + 1]);
            const float q = (float)((packed[i / 2] >> (4 * (i & 1))) & 0x0f);
            volatile float prod = s * q; /* volatile: no contraction into an fma */
            dense[i] = prod + b;
        }
    }
}

/* y[m, row] = sum_c dense[row, c] * x[m, c] accumulated in f64 and rounded to
 * f32 once: the "dequant-matvec" the reference's tests compare kernels with
 * (tests/common/mod.rs:550-556). x holds bf16 bit patterns. threads <= 0 uses
 * every core. */
ORC_API void orc_q4_dense_gemm(const uint8_t *packed, const uint16_t *sb, const uint16_t *x_bf16, size_t m,
                               size_t rows, size_t cols, size_t group, float *y, int threads)
{
    const size_t gpr = cols / group;
    float *xf = (float *)malloc(sizeof(float) * m * cols);
    for (size_t i = 0; i < m * cols; ++i) xf[i] = orc_bf16_bits_to_f32(x_bf16[i]);
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        double acc[64];
        for (size_t m0 = 0; m0 < m; m0 += 64) {
            const size_t mc = (m - m0) < 64 ? (m - m0) : 64;
            for (size_t j = 0; j < mc; ++j) acc[j] = 0.0;
            for (size_t c = 0; c < cols; ++c) {
                const size_t i = (size_t)r * cols + c;
                const size_t gi = (size_t)r * gpr + c / group;
                const float s = orc_bf16_bits_to_f32(sb[2 * gi]);
                const float b = orc_bf16_bits_to_f32(sb[2 * gi + 1]);
                const float q = (float)((packed[i / 2] >> (4 * (i & 1))) & 0x0f);
                volatile float prod = s * q;
                const double w = (double)(float)(prod + b);
                for (size_t j = 0; j < mc; ++j) acc[j] += w * (double)xf[(m0 + j) * cols + c];
            }
            for (size_t j = 0; j < mc; ++j) y[(m0 + j) * rows + (size_t)r] = (float)acc[j];
        }
    }
    free(xf);
}

/* The affine product in f64 without the dequant rounding, and the magnitude
 * S = sum_g |s| sum|q x| + |b| sum|x| that scales the reference's derived
 * bound gamma_t * S (tests/gemm_q4_mlx_tensorops.rs:33-64). mag may be NULL. */
ORC_API void orc_q4_affine_gemm_f64(const uint8_t *packed, const uint16_t *sb, const uint16_t *x_bf16, size_t m,
                                    size_t rows, size_t cols, size_t group, double *want, double *mag,
                                    int threads)
{
    const size_t gpr = cols / group;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (ptrdiff_t ni = 0; ni < (ptrdiff_t)rows; ++ni) {
        for (size_t mi = 0; mi < m; ++mi) {
            double acc = 0.0, s_mag = 0.0;
            for (size_t g = 0; g < gpr; ++g) {
                const double s = (double)orc_bf16_bits_to_f32(sb[2 * ((size_t)ni * gpr + g)]);
                const double b = (double)orc_bf16_bits_to_f32(sb[2 * ((size_t)ni * gpr + g) + 1]);
                double qx = 0.0, aqx = 0.0, xsum = 0.0, ax = 0.0;
                for (size_t j = 0; j < group; ++j) {
                    const size_t i = (size_t)ni * cols + g * group + j;
                    const double xv = (double)orc_bf16_bits_to_f32(x_bf16[mi * cols + g * group + j]);
                    const double q = (double)((packed[i / 2] >> (4 * (i & 1))) & 0x0f);
                    qx += q * xv;
                    aqx += q * fabs(xv);
                    xsum += xv;
                    ax += fabs(xv);
                }
                acc += s * qx + b * xsum;
                s_mag += fabs(s) * aqx + fabs(b) * ax;
            }
            want[mi * rows + (size_t)ni] = acc;
            if (mag) mag[mi * rows + (size_t)ni] = s_mag;
        }
    }
}

/* gamma_t = t u / (1 - t u), u = 2^-24 (tests/gemm_q4_mlx_tensorops.rs:66-69). */
ORC_API double orc_gamma(size_t terms)
{
    const double tu = (double)terms * ldexp(1.0, -24);
    return tu / (1.0 - tu);
}

/* numcheck's reduction tolerance 4 * eps_f32 * sqrt(n) * scale
 * (numcheck/src/lib.rs:164-166). */
ORC_API double orc_reduction_tolerance(size_t n, double scale)
{
    return 4.0 * (double)1.1920928955078125e-07f * sqrt((double)n) * scale;
}

/* ---------------------------------------------------------- activations --- */

/* f64 SiLU with the sign-branching sigmoid (tests/common/mod.rs:571-588). */
ORC_API double orc_silu_f64(double x)
{
    double sg;
    if (x >= 0.0) {
        sg = 1.0 / (1.0 + exp(-x));
    } else {
        const double e = exp(x);
        sg = e / (1.0 + e);
    }
    return x * sg;
}

/* f64 tanh-approximate GELU, cubic input clamped to +-20, tanh argument to
 * +-10, outer factor the original x (tests/common/mod.rs:558-569). */
ORC_API double orc_gelu_f64(double x)
{
    double xc = x < -20.0 ? -20.0 : (x > 20.0 ? 20.0 : x);
    double inner = 0.7978845608028654 * (xc + 0.044715 * xc * xc * xc);
    inner = inner < -10.0 ? -10.0 : (inner > 10.0 ? 10.0 : inner);
    return 0.5 * x * (1.0 + tanh(inner));
}

/* The kernels' own f32 SiLU: e = exp(-|x|), r = 1/(1+e), sigmoid = x>=0 ? r
 * : e*r (kernels/act.h:36-46). */
ORC_API float orc_silu_f32(float x)
{
    const float e = expf(-fabsf(x));
    const float r = 1.0f / (1.0f + e);
    const float sg = x >= 0.0f ? r : e * r;
    return x * sg;
}

/* The kernels' own f32 GELU (kernels/act.h:24-30). */
ORC_API float orc_gelu_f32(float x)
{
    float xc = x < -20.0f ? -20.0f : (x > 20.0f ? 20.0f : x);
    const float x3 = xc * xc * xc;
    float inner = 0.7978845608028654f * (xc + 0.044715f * x3);
    inner = inner < -10.0f ? -10.0f : (inner > 10.0f ? 10.0f : inner);
    const float t = tanhf(inner);
    return 0.5f * x * (1.0f + t);
}

/* ------------------------------------------- order-faithful Q4 kernels --- */

/* Knobs for what the Metal compiler is free to choose under fast math, so the
 * pin test can find the combination the recorded words were produced with:
 *   sum_mode    0: simd_sum as a shuffle-down tree (w = 16, 8, 4, 2, 1)
 *               1: xor butterfly (every lane ends with the same value)
 *               2: serial lane 0..31
 *               3: xor butterfly with ascending strides 1, 2, 4, 8, 16: adjacent
 *                  lanes first (the order the recorded outputs follow)
 *   affine_mode 0: scale*accum and xsum*bias rounded separately, added, then
 *                  added to the lane's running sum
 *               1: fma(scale, accum, xsum*bias), then added to the running sum
 *               2: fma(xsum, bias, scale*accum), then added to the running sum
 *               3: fma(scale, accum, fma(xsum, bias, running sum))
 *               4: fma(xsum, bias, fma(scale, accum, running sum))
 *   chain_mode  0: accum += ((e0+e1)+e2)+e3 as the source groups it
 *               1: accum = (((accum+e0)+e1)+e2)+e3
 */
typedef struct {
    int sum_mode;
    int affine_mode;
    int chain_mode;
} OrcOrder;

static float simd_sum_emul(const float *lane_vals, int sum_mode)
{
    float buf[32];
    memcpy(buf, lane_vals, sizeof buf);
    if (sum_mode == 2) {
        float s = buf[0];
        for (int i = 1; i < 32; ++i) s += buf[i];
        return s;
    }
    if (sum_mode == 3) {
        for (int w = 1; w < 32; w <<= 1) {
            float nxt[32];
            for (int i = 0; i < 32; ++i) nxt[i] = buf[i] + buf[i ^ w];
            memcpy(buf, nxt, sizeof buf);
        }
        return buf[0];
    }
    if (sum_mode == 1) {
        for (int w = 16; w > 0; w >>= 1) {
            float nxt[32];
            for (int i = 0; i < 32; ++i) nxt[i] = buf[i] + buf[i ^ w];
            memcpy(buf, nxt, sizeof buf);
        }
        return buf[0];
    }
    for (int w = 16; w > 0; w >>= 1)
        for (int i = 0; i < w; ++i) buf[i] += buf[i + w];
    return buf[0];
}

/* load_x16_qdot: 16 bf16 activations widened, their sum, and the 16^-k
 * prescale (kernels/q4_mlx_dot.h:44-62). */
static float load_x16(const uint16_t *x, float *xp)
{
    float a[16];
    for (int i = 0; i < 16; ++i) a[i] = orc_bf16_bits_to_f32(x[i]);
    const float sum = (((a[0] + a[1]) + a[2]) + a[3]) + (((a[4] + a[5]) + a[6]) + a[7]) +
                      (((a[8] + a[9]) + a[10]) + a[11]) + (((a[12] + a[13]) + a[14]) + a[15]);
    static const float inv[4] = {1.0f, 1.0f / 16.0f, 1.0f / 256.0f, 1.0f / 4096.0f};
    for (int i = 0; i < 16; ++i) xp[i] = a[i] * inv[i & 3]; /* exact: a power of two */
    return sum;
}

/* qdot16: sixteen nibbles masked in place against the prescaled x, then
 * scale * accum + xsum * bias (kernels/q4_mlx_dot.h:72-94). */
static float qdot16_emul(const uint8_t *w, const float *xp, float scale, float bias, float xsum, OrcOrder o,
                         float acc_in)
{
    uint32_t w2[2];
    memcpy(w2, w, 8);
    const uint32_t ww[4] = {w2[0] & 0xffffu, w2[0] >> 16, w2[1] & 0xffffu, w2[1] >> 16};
    static const uint32_t mask[4] = {0x000fu, 0x00f0u, 0x0f00u, 0xf000u};
    volatile float accum = 0.0f;
    for (int j = 0; j < 4; ++j) {
        volatile float e[4];
        for (int i = 0; i < 4; ++i) e[i] = xp[4 * j + i] * (float)(ww[j] & mask[i]);
        if (o.chain_mode == 0) {
            volatile float t = e[0] + e[1];
            t = t + e[2];
            t = t + e[3];
            accum = accum + t;
        } else {
            accum = accum + e[0];
            accum = accum + e[1];
            accum = accum + e[2];
            accum = accum + e[3];
        }
    }
    volatile float sa = scale * accum;
    volatile float xb = xsum * bias;
    volatile float t;
    switch (o.affine_mode) {
    case 1: t = fmaf(scale, accum, xb); return acc_in + t;
    case 2: t = fmaf(xsum, bias, sa); return acc_in + t;
    case 3: t = fmaf(xsum, bias, acc_in); return fmaf(scale, accum, t);
    case 4: t = fmaf(scale, accum, acc_in); return fmaf(xsum, bias, t);
    default: t = sa + xb; return acc_in + t;
    }
}

enum { ORC_EPI_STORE = 0, ORC_EPI_ADD_RESID = 1, ORC_EPI_GATE_UP_GELU = 2, ORC_EPI_GATE_UP_SILU = 3 };

/* q4_simd_gemv for the row-major layout: one simdgroup owns four rows, each
 * lane sixteen columns of every 512-column block, f32 partial sums per lane,
 * simd_sum per row, then the epilogue (kernels/gemv_q4_mlx_simd.h:114-213).
 * out receives f32 words, or bf16 halves packed two per word position when
 * mid_as_bf16 is set for a gate/up epilogue. bank1 is read only by the
 * gate/up epilogues, resid only by ADD_RESID. Rows past `rows` are never
 * written. */
ORC_API void orc_q4_simd_gemv(const uint8_t *packed0, const uint16_t *sb0, const uint8_t *packed1,
                              const uint16_t *sb1, const uint16_t *x_bf16, void *out, const float *resid,
                              int epi, int mid_as_bf16, uint32_t rows, uint32_t cols, uint32_t group,
                              int sum_mode, int affine_mode, int chain_mode, int threads)
{
    const OrcOrder o = {sum_mode, affine_mode, chain_mode};
    const int nb = (epi == ORC_EPI_GATE_UP_GELU || epi == ORC_EPI_GATE_UP_SILU) ? 2 : 1;
    const uint8_t *packed[2] = {packed0, packed1};
    const uint16_t *sbs[2] = {sb0, sb1};
    const uint32_t gpr = cols / group;
    const size_t row_bytes = cols >> 1;
    const ptrdiff_t n_sg = (ptrdiff_t)((rows + 3u) / 4u);
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (ptrdiff_t sg = 0; sg < n_sg; ++sg) {
        const uint32_t row0 = (uint32_t)sg * 4u;
        float acc[2][4][32];
        memset(acc, 0, sizeof acc);
        for (uint32_t lane = 0; lane < 32u; ++lane) {
            const uint32_t lane_col0 = lane * 16u;
            for (uint64_t k0 = 0; k0 < cols; k0 += 512u) {
                const uint64_t col = k0 + lane_col0;
                if (col + 16u > cols) continue;
                float xp[16];
                const float xsum = load_x16(x_bf16 + col, xp);
                for (uint32_t r = 0; r < 4u; ++r) {
                    if (row0 + r >= rows) break;
                    for (int b = 0; b < nb; ++b) {
                        const size_t gi = (size_t)(row0 + r) * gpr + col / group;
                        const float s = orc_bf16_bits_to_f32(sbs[b][2 * gi]);
                        const float bi = orc_bf16_bits_to_f32(sbs[b][2 * gi + 1]);
                        const uint8_t *wp = packed[b] + (size_t)(row0 + r) * row_bytes + (col >> 1);
                        acc[b][r][lane] = qdot16_emul(wp, xp, s, bi, xsum, o, acc[b][r][lane]);
                    }
                }
            }
        }
        for (uint32_t r = 0; r < 4u; ++r) {
            const uint32_t row = row0 + r;
            if (row >= rows) break;
            float sum[2];
            for (int b = 0; b < nb; ++b) sum[b] = simd_sum_emul(acc[b][r], o.sum_mode);
            if (epi == ORC_EPI_STORE) {
                ((float *)out)[row] = sum[0];
            } else if (epi == ORC_EPI_ADD_RESID) {
                ((float *)out)[row] = sum[0] + resid[row];
            } else {
                const float act = (epi == ORC_EPI_GATE_UP_SILU) ? orc_silu_f32(sum[0]) : orc_gelu_f32(sum[0]);
                const float v = act * sum[nb - 1];
                if (mid_as_bf16) {
                    ((uint16_t *)out)[row] = orc_f32_to_bf16_bits_gpu(v);
                } else {
                    ((float *)out)[row] = v;
                }
            }
        }
    }
}

/* q4_simd_gemm for the row-major layout: the same lane structure with up to
 * eight activation rows carried through one weight read; y[m * rows + row]
 * (kernels/gemm_q4_mlx_simd.h:29-100). */
ORC_API void orc_q4_simd_gemm(const uint8_t *packed, const uint16_t *sb, const uint16_t *x_bf16, float *y,
                              const float *resid, uint32_t rows, uint32_t cols, uint32_t group, uint32_t m,
                              int sum_mode, int affine_mode, int chain_mode, int threads)
{
    const OrcOrder o = {sum_mode, affine_mode, chain_mode};
    const uint32_t m_cap = m < 8u ? m : 8u;
    if (m_cap == 0) return;
    const uint32_t gpr = cols / group;
    const size_t row_bytes = cols >> 1;
    const ptrdiff_t n_sg = (ptrdiff_t)((rows + 3u) / 4u);
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (ptrdiff_t sg = 0; sg < n_sg; ++sg) {
        const uint32_t row0 = (uint32_t)sg * 4u;
        float acc[4][8][32];
        memset(acc, 0, sizeof acc);
        for (uint32_t lane = 0; lane < 32u; ++lane) {
            const uint32_t lane_col0 = lane * 16u;
            for (uint64_t k0 = 0; k0 < cols; k0 += 512u) {
                const uint64_t col = k0 + lane_col0;
                if (col + 16u > cols) continue;
                float xt[8][16];
                float xsum[8];
                for (uint32_t mi = 0; mi < m_cap; ++mi) xsum[mi] = load_x16(x_bf16 + (size_t)mi * cols + col, xt[mi]);
                for (uint32_t r = 0; r < 4u; ++r) {
                    const uint32_t row = row0 + r;
                    if (row >= rows) break;
                    const size_t gi = (size_t)row * gpr + col / group;
                    const float s = orc_bf16_bits_to_f32(sb[2 * gi]);
                    const float bi = orc_bf16_bits_to_f32(sb[2 * gi + 1]);
                    const uint8_t *wp = packed + (size_t)row * row_bytes + (col >> 1);
                    for (uint32_t mi = 0; mi < m_cap; ++mi) {
                        acc[r][mi][lane] = qdot16_emul(wp, xt[mi], s, bi, xsum[mi], o, acc[r][mi][lane]);
                    }
                }
            }
        }
        for (uint32_t r = 0; r < 4u; ++r) {
            const uint32_t row = row0 + r;
            if (row >= rows) break;
            for (uint32_t mi = 0; mi < m_cap; ++mi) {
                const float sum = simd_sum_emul(acc[r][mi], o.sum_mode);
                const size_t idx = (size_t)mi * rows + row;
                y[idx] = resid ? sum + resid[idx] : sum;
            }
        }
    }
}

/* ------------------------------------------------------------------- Q8 --- */

/* f64 reference of the Q8 GEMV: w = scale * (q - zero), signed int8 codes,
 * f32 scales and zeros per group, f32 x (tests/quantized_gemv.rs:103-124). */
ORC_API void orc_q8_gemv_f64(const int8_t *q, const float *scales, const float *zeros, const float *x,
                             size_t rows, size_t cols, size_t group, float *y, int threads)
{
    const size_t gpr = cols / group;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        double acc = 0.0;
        for (size_t c = 0; c < cols; ++c) {
            const size_t g = (size_t)r * gpr + c / group;
            const double w = (double)scales[g] * ((double)q[(size_t)r * cols + c] - (double)zeros[g]);
            acc += w * (double)x[c];
        }
        y[r] = (float)acc;
    }
}

/* The Q8 kernel's own f32 order: group-major, four columns per lane per step
 * when the group is a multiple of four, prod = w * x summed as
 * (p.x + p.y) + (p.z + p.w), simd_sum per row (kernels/gemv_q8.metal:33-122). */
ORC_API void orc_q8_simd_gemv(const int8_t *q, const float *scales, const float *zeros, const float *x,
                              uint32_t rows, uint32_t cols, uint32_t group, float *y, int sum_mode, int threads)
{
    const uint32_t gpr = cols / group;
    const int vec4_ok = (group % 4u == 0u) && (cols % 4u == 0u);
    const ptrdiff_t n_sg = (ptrdiff_t)((rows + 3u) / 4u);
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (ptrdiff_t sg = 0; sg < n_sg; ++sg) {
        const uint32_t row0 = (uint32_t)sg * 4u;
        float acc[4][32];
        memset(acc, 0, sizeof acc);
        for (uint32_t lane = 0; lane < 32u; ++lane) {
            for (uint32_t g = 0; g < gpr; ++g) {
                const uint64_t c0 = (uint64_t)g * group;
                for (uint32_t r = 0; r < 4u; ++r) {
                    const uint32_t row = row0 + r;
                    if (row >= rows) break;
                    const float s = scales[(size_t)row * gpr + g];
                    const float z = zeros[(size_t)row * gpr + g];
                    if (vec4_ok) {
                        for (uint64_t i = (uint64_t)lane * 4u; i < group; i += 128u) {
                            const uint64_t c = c0 + i;
                            volatile float p[4];
                            for (int j = 0; j < 4; ++j) {
                                volatile float d = (float)q[(size_t)row * cols + c + j] - z;
                                volatile float w = s * d;
                                p[j] = w * x[c + j];
                            }
                            volatile float a = p[0] + p[1];
                            volatile float b = p[2] + p[3];
                            volatile float t = a + b;
                            acc[r][lane] = acc[r][lane] + t;
                        }
                    } else {
                        for (uint64_t i = lane; i < group; i += 32u) {
                            volatile float d = (float)q[(size_t)row * cols + c0 + i] - z;
                            volatile float w = s * d;
                            volatile float p = w * x[c0 + i];
                            acc[r][lane] = acc[r][lane] + p;
                        }
                    }
                }
            }
        }
        for (uint32_t r = 0; r < 4u; ++r) {
            const uint32_t row = row0 + r;
            if (row < rows) y[row] = simd_sum_emul(acc[r], sum_mode);
        }
    }
}

/* MLX-layout Q8 (unsigned codes 0..255, bf16 (scale, bias) pairs, bf16 x):
 * w = scale * code + bias dequantized in f32 with a separate multiply and
 * add, then the f64 matvec. The reference has no kernel for this layout; it
 * is the Q4 dequant-matvec rule (tests/common/mod.rs:528-556) applied to
 * 8-bit codes, and for bias = -128 * scale it equals orc_q8_gemv_f64 on
 * code - 128 with zero = 0. */
ORC_API void orc_q8_mlx_dense_gemm(const uint8_t *codes, const uint16_t *sb, const uint16_t *x_bf16, size_t m,
                                   size_t rows, size_t cols, size_t group, float *y, int threads)
{
    const size_t gpr = cols / group;
    float *xf = (float *)malloc(sizeof(float) * m * cols);
    for (size_t i = 0; i < m * cols; ++i) xf[i] = orc_bf16_bits_to_f32(x_bf16[i]);
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r) {
        double acc[8];
        for (size_t m0 = 0; m0 < m; m0 += 8) {
            const size_t mc = (m - m0) < 8 ? (m - m0) : 8;
            for (size_t j = 0; j < mc; ++j) acc[j] = 0.0;
            for (size_t c = 0; c < cols; ++c) {
                const size_t gi = (size_t)r * gpr + c / group;
                const float s = orc_bf16_bits_to_f32(sb[2 * gi]);
                const float b = orc_bf16_bits_to_f32(sb[2 * gi + 1]);
                volatile float prod = s * (float)codes[(size_t)r * cols + c];
                const double w = (double)(float)(prod + b);
                for (size_t j = 0; j < mc; ++j) acc[j] += w * (double)xf[(m0 + j) * cols + c];
            }
            for (size_t j = 0; j < mc; ++j) y[(m0 + j) * rows + (size_t)r] = (float)acc[j];
        }
    }
    free(xf);
}

/* Dense f32 image of an MLX-layout Q8 bank (same rule as orc_q4_dequant). */
ORC_API void orc_q8_mlx_dequant(const uint8_t *codes, const uint16_t *sb, size_t rows, size_t cols, size_t group,
                                float *dense)
{
    const size_t gpr = cols / group;
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) {
            const size_t gi = r * gpr + c / group;
            volatile float prod = orc_bf16_bits_to_f32(sb[2 * gi]) * (float)codes[r * cols + c];
            dense[r * cols + c] = prod + orc_bf16_bits_to_f32(sb[2 * gi + 1]);
        }
}

/* --------------------------------------------------------------- hashing --- */

/* FNV-1a over the little-endian bytes of 32-bit words, the hash the
 * reference's known-answer table records (tests/q4_kernels_template.rs:55-64). */
ORC_API uint64_t orc_fnv1a_words(const uint32_t *words, size_t n)
{
    uint64_t h = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < n; ++i) {
        for (int b = 0; b < 4; ++b) {
            h ^= (uint64_t)((words[i] >> (8 * b)) & 0xffu);
            h *= 0x00000100000001b3ull;
        }
    }
    return h;
}

ORC_API int orc_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
