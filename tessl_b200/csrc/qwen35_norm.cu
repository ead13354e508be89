// The steps either side of a projection in Qwen3.5 decode: the zero-centred RMSNorm that produces
// the bf16 activations a Q4 projection reads, the residual add, and the two in one launch.
//
// Mirrors `qwen35::rms_norm`, `qwen35::residual_add` and `qwen35::add_rms_norm`
// (src/qwen35.rs:2586-2755 of the reference project) and their kernels
// (kernels/qwen35_mlp.metal:53-171): out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * (1 + w[:]),
// f32 in, f32 or bf16 out, `1 + w` formed in f32 here. The fused form adds y into resid first and is
// bit-identical to the two separate calls: the add is the same f32 add, every element is read back by
// the thread that wrote it, and the sum of squares is reduced in the same order by the same code.
//
// One block of 256 threads per row; each thread walks the row in float4 steps of the block's width.
// The rows are a few KB, so the kernels are launch-bound; they are launched with programmatic stream
// serialization so that a following GEMV can already stream its weights while they run.
#include "q4_common.cuh"
#include "runtime.h"

namespace tessl {
namespace {

constexpr int kNormThreads = 256;

/// Sum over the block, the same value in every thread: lanes by xor butterfly, then the warps' sums in
/// warp order by every thread.
__device__ __forceinline__ float block_sum(float v, float *scratch)
{
    v = dev::warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += scratch[w];
    return total;
}

template <bool ADD, bool OUT_BF16>
__global__ void __launch_bounds__(kNormThreads) qwen35_rms_norm_kernel(const float *y, float *x_or_resid, const float *weight,
                                                                      void *out, uint32_t dim, float eps)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float scratch[kNormThreads / 32];
    const size_t base = (size_t)blockIdx.x * dim;
    float *xr = x_or_resid + base;
    const float *yr = ADD ? y + base : nullptr;
    float ss = 0.0f;
    const bool vec = (dim & 3u) == 0;  // rows start 16-byte aligned then (the wrappers check the buffers)
    if (vec) {
        for (uint32_t d = threadIdx.x * 4; d < dim; d += kNormThreads * 4) {
            float4 v = *reinterpret_cast<const float4 *>(xr + d);
            if constexpr (ADD) {
                const float4 a = *reinterpret_cast<const float4 *>(yr + d);
                v.x = v.x + a.x, v.y = v.y + a.y, v.z = v.z + a.z, v.w = v.w + a.w;
                *reinterpret_cast<float4 *>(xr + d) = v;
            }
            ss = fmaf(v.x, v.x, ss), ss = fmaf(v.y, v.y, ss), ss = fmaf(v.z, v.z, ss), ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (uint32_t d = threadIdx.x; d < dim; d += kNormThreads) {
            float v = xr[d];
            if constexpr (ADD) {
                v = v + yr[d];
                xr[d] = v;
            }
            ss = fmaf(v, v, ss);
        }
    }
    const float mean = __fdiv_rn(block_sum(ss, scratch), (float)dim);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(mean + eps));
    auto store = [&](uint32_t d, float v) {
        const float o = __fmul_rn(__fmul_rn(v, inv), 1.0f + weight[d]);
        if constexpr (OUT_BF16) {
            static_cast<uint16_t *>(out)[base + d] = dev::f32_to_bf16_store(o);
        } else {
            static_cast<float *>(out)[base + d] = o;
        }
    };
    if (vec) {
        for (uint32_t d = threadIdx.x * 4; d < dim; d += kNormThreads * 4) {
            const float4 v = *reinterpret_cast<const float4 *>(xr + d);  // its own writes, if ADD
            store(d, v.x), store(d + 1, v.y), store(d + 2, v.z), store(d + 3, v.w);
        }
    } else {
        for (uint32_t d = threadIdx.x; d < dim; d += kNormThreads) store(d, xr[d]);
    }
}

__global__ void qwen35_residual_add_kernel(const float *y, float *resid, uint64_t n)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) resid[i] = resid[i] + y[i];
}

template <typename K, typename... A>
Result launch_pdl(TesslRuntime *rt, K kernel, dim3 grid, dim3 block, const char *what, A... args)
{
    cudaLaunchConfig_t lc{};
    lc.gridDim = grid, lc.blockDim = block, lc.dynamicSmemBytes = 0, lc.stream = rt->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr, lc.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&lc, kernel, args...);
    rt->dispatch_count += 1;
    return cuda_check(rt, e, what);
}

/// `nn::validate_rms_scalars` (src/nn.rs:190-202 of the reference project).
Result validate_rms_scalars(uint32_t dim, float eps, const char *what)
{
    if (dim == 0) return fmt("%s: dim must be non-zero", what);
    if (!(eps > 0.0f) || !(eps < 3.0e38f)) return fmt("%s: eps must be finite and positive", what);
    return ok();
}

Result require_aligned4(const TesslBuf &b, const char *what)
{
    if (((uintptr_t)b.ptr & 15u) != 0) return fmt("%s: device pointer must be 16-byte aligned", what);
    return ok();
}

}  // namespace

namespace nn {

Result qwen35_rms_norm(TesslRuntime *rt, const TesslBuf &x, const TesslBuf &w, const TesslBuf &out, bool out_as_bf16,
                       uint32_t rows, uint32_t dim, float eps)
{
    const char *what = "qwen35::rms_norm";
    TESSL_TRY(validate_rms_scalars(dim, eps, what));
    const uint64_t n = elems(rows, dim);
    TESSL_TRY(require(x, n, 4, "rms_norm x"));
    TESSL_TRY(require(w, dim, 4, "rms_norm w"));
    TESSL_TRY(require(out, n, out_as_bf16 ? 2 : 4, "rms_norm out"));
    if (rows == 0) return ok();
    const Named writes[] = {{"out", &out}};
    if (out_as_bf16) {
        const Named reads[] = {{"x", &x}, {"w", &w}};
        TESSL_TRY(require_disjoint_writes(what, writes, 1, reads, 2));
    } else {
        // an f32 output may be x itself: every element is read and written by the same thread
        const Named reads[] = {{"w", &w}};
        TESSL_TRY(require_disjoint_writes(what, writes, 1, reads, 1));
        if (aliases(out, x) && out.ptr != x.ptr) return fmt("%s: out overlaps x without being x", what);
    }
    TESSL_TRY(require_aligned4(x, "rms_norm x"));
    TESSL_TRY(require_aligned4(out, "rms_norm out"));
    float *xp = static_cast<float *>(x.ptr);
    const float *wp = static_cast<const float *>(w.ptr);
    if (out_as_bf16)
        return launch_pdl(rt, qwen35_rms_norm_kernel<false, true>, dim3(rows), dim3(kNormThreads), "qwen35_rms_norm launch",
                          (const float *)nullptr, xp, wp, out.ptr, dim, eps);
    return launch_pdl(rt, qwen35_rms_norm_kernel<false, false>, dim3(rows), dim3(kNormThreads), "qwen35_rms_norm launch",
                      (const float *)nullptr, xp, wp, out.ptr, dim, eps);
}

Result qwen35_residual_add(TesslRuntime *rt, const TesslBuf &y, const TesslBuf &resid, uint32_t rows, uint32_t width)
{
    const char *what = "qwen35::residual_add";
    const uint64_t n = elems(rows, width);
    TESSL_TRY(require(y, n, 4, "residual_add y"));
    TESSL_TRY(require(resid, n, 4, "residual_add resid"));
    if (n == 0) return ok();
    const Named writes[] = {{"resid", &resid}};
    const Named reads[] = {{"y", &y}};
    TESSL_TRY(require_disjoint_writes(what, writes, 1, reads, 1));
    return launch_pdl(rt, qwen35_residual_add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256),
                      "qwen35_residual_add launch", static_cast<const float *>(y.ptr), static_cast<float *>(resid.ptr), n);
}

Result qwen35_add_rms_norm(TesslRuntime *rt, const TesslBuf &y, const TesslBuf &resid, const TesslBuf &w, const TesslBuf &out,
                           bool out_as_bf16, uint32_t rows, uint32_t dim, float eps)
{
    const char *what = "qwen35::add_rms_norm";
    TESSL_TRY(validate_rms_scalars(dim, eps, what));
    const uint64_t n = elems(rows, dim);
    TESSL_TRY(require(y, n, 4, "add_rms_norm y"));
    TESSL_TRY(require(resid, n, 4, "add_rms_norm resid"));
    TESSL_TRY(require(w, dim, 4, "add_rms_norm w"));
    TESSL_TRY(require(out, n, out_as_bf16 ? 2 : 4, "add_rms_norm out"));
    if (rows == 0) return ok();
    const Named writes[] = {{"resid", &resid}, {"out", &out}};
    const Named reads[] = {{"y", &y}, {"w", &w}};
    TESSL_TRY(require_disjoint_writes(what, writes, 2, reads, 2));
    TESSL_TRY(require_aligned4(y, "add_rms_norm y"));
    TESSL_TRY(require_aligned4(resid, "add_rms_norm resid"));
    TESSL_TRY(require_aligned4(out, "add_rms_norm out"));
    const float *yp = static_cast<const float *>(y.ptr), *wp = static_cast<const float *>(w.ptr);
    float *rp = static_cast<float *>(resid.ptr);
    if (out_as_bf16)
        return launch_pdl(rt, qwen35_rms_norm_kernel<true, true>, dim3(rows), dim3(kNormThreads), "qwen35_add_rms_norm launch",
                          yp, rp, wp, out.ptr, dim, eps);
    return launch_pdl(rt, qwen35_rms_norm_kernel<true, false>, dim3(rows), dim3(kNormThreads), "qwen35_add_rms_norm launch", yp,
                      rp, wp, out.ptr, dim, eps);
}

}  // namespace nn
}  // namespace tessl
