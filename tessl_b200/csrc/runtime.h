// Runtime handle and host-side validation helpers shared by the operator files.
//
// The handle is the thin CUDA analogue of the reference's `GpuRuntime`
// (src/runtime.rs): a device ordinal, one stream, a poison latch, a launch
// counter and a growable scratch allocation. The helpers restate the refusal
// rules of `src/nn.rs` (`require`, `require_disjoint_writes`, `QuantShape::validate`,
// `Q4MlxBank::validate`) with the same wording, so a caller switching libraries
// sees the same messages.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <thread>

#include "../../include/tessl_b200.h"

namespace tessl {

/// Empty string = Ok(()); anything else is the Err(String) message.
using Result = std::string;
inline Result ok() { return std::string(); }

template <typename... A>
inline std::string fmt(const char *f, A... a)
{
    char buf[768];
    std::snprintf(buf, sizeof buf, f, a...);
    return std::string(buf);
}

}  // namespace tessl

struct TesslRuntime {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::thread::id owner;
    bool poisoned = false;
    bool async_encode = false;
    bool encode_only = false;
    uint64_t dispatch_count = 0;
    int sm_count = 148;
    // Scratch for kernels that need global memory beyond their operands
    // (split-K partial sums, the prefill GEMM's converted activations). Grown on
    // demand, never shrunk, freed with the handle.
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    void *tensormap_encode = nullptr;  // cuTensorMapEncodeTiled, resolved lazily
    // One word of pinned host memory a kernel writes (through its device
    // alias) when a bounded wait inside it gives up. Checked at every wait.
    volatile uint32_t *status_host = nullptr;
    uint32_t *status_dev = nullptr;
    // Dynamic shared memory already opted in, per kernel. The attribute belongs to the
    // device's context, so it is remembered per runtime (one device each), not per process.
    std::map<const void *, size_t> smem_opted;
    // Prefill GEMM tile choice: what a tuning run or a test asked for (0 / -1 = the library
    // decides) and what the last call ran (0 = no tile kernel ran, e.g. the small-batch route).
    int prefill_force_bn = 0;
    int prefill_force_pair = -1;
    int prefill_last_bn = 0;
    int prefill_last_pair = 0;
    // Clock budget of a bounded device-side wait on another rank (0 = the default).
    uint64_t peer_wait_clocks = 0;
};

namespace tessl {

/// Latches the poison flag on a CUDA error and turns it into a message.
inline Result cuda_check(TesslRuntime *rt, cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return ok();
    if (rt) rt->poisoned = true;
    return fmt("%s: CUDA error %d (%s); the runtime is poisoned and must be recreated", what, (int)e,
               cudaGetErrorString(e));
}

/// Opts `kernel` in to `bytes` of dynamic shared memory on the runtime's device, once per
/// runtime and size; `carveout` also asks for the largest shared-memory carve-out.
inline Result smem_opt_in(TesslRuntime *rt, const void *kernel, size_t bytes, const char *what, bool carveout = false)
{
    auto it = rt->smem_opted.find(kernel);
    if (it != rt->smem_opted.end() && it->second >= bytes) return ok();
    Result r = cuda_check(rt, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), what);
    if (!r.empty()) return r;
    if (carveout) {
        r = cuda_check(rt, cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                (int)cudaSharedmemCarveoutMaxShared), what);
        if (!r.empty()) return r;
    }
    rt->smem_opted[kernel] = bytes;
    return ok();
}

/// Scratch of at least `bytes`, 256-byte aligned. Growing waits for the stream
/// (earlier kernels may still read the old allocation) and reallocates.
inline Result scratch_reserve(TesslRuntime *rt, size_t bytes, void **out)
{
    if (bytes > rt->scratch_bytes) {
        Result r = cuda_check(rt, cudaStreamSynchronize(rt->stream), "scratch_reserve: synchronize");
        if (!r.empty()) return r;
        if (rt->scratch) cudaFree(rt->scratch);
        rt->scratch = nullptr;
        rt->scratch_bytes = 0;
        size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
        cudaError_t e = cudaMalloc(&rt->scratch, want);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fmt("scratch_reserve: cannot allocate %zu bytes of scratch (%s)", want, cudaGetErrorString(e));
        }
        rt->scratch_bytes = want;
    }
    *out = rt->scratch;
    return ok();
}

// ------------------------------------------------------------ validation ---

inline uint64_t elems(uint32_t a, uint32_t b) { return uint64_t(a) * uint64_t(b); }

/// `nn::require::<T>` (src/nn.rs:126-143): capacity in elements of `elem` bytes.
inline Result require(const TesslBuf &buf, uint64_t need, size_t elem, const std::string &what)
{
    const uint64_t have = buf.nbytes / elem;
    if (have < need) {
        return fmt("%s: buffer holds %llu elements, kernel reads/writes %llu", what.c_str(),
                   (unsigned long long)have, (unsigned long long)need);
    }
    if (need > 0 && buf.ptr == nullptr) return fmt("%s: null device pointer", what.c_str());
    return ok();
}

inline bool aliases(const TesslBuf &a, const TesslBuf &b)
{
    if (!a.ptr || !b.ptr || a.nbytes == 0 || b.nbytes == 0) return false;
    const uintptr_t a0 = (uintptr_t)a.ptr, a1 = a0 + a.nbytes, b0 = (uintptr_t)b.ptr, b1 = b0 + b.nbytes;
    return a0 < b1 && b0 < a1;
}

struct Named {
    const char *name;
    const TesslBuf *buf;
};

/// `nn::require_disjoint_writes` (src/nn.rs:146-187): no writable buffer may
/// overlap another writable buffer or any read-only one.
inline Result require_disjoint_writes(const char *entry, const Named *writes, int nw, const Named *reads, int nr)
{
    for (int i = 0; i < nw; ++i) {
        for (int j = i + 1; j < nw; ++j) {
            if (aliases(*writes[i].buf, *writes[j].buf))
                return fmt("%s: writable buffers %s and %s overlap", entry, writes[i].name, writes[j].name);
        }
        for (int j = 0; j < nr; ++j) {
            if (aliases(*writes[i].buf, *reads[j].buf))
                return fmt("%s: writable buffer %s overlaps read-only buffer %s", entry, writes[i].name,
                           reads[j].name);
        }
    }
    return ok();
}

/// `QuantShape::validate` (src/nn.rs:3254-3267).
inline Result quant_shape_validate(const TesslQuantShape &s, const std::string &what)
{
    if (s.group_size == 0) return fmt("%s: group_size must be non-zero", what.c_str());
    if (s.cols % s.group_size != 0) {
        return fmt("%s: cols %u is not a multiple of group_size %u; the kernels compute `cols / group_size` "
                   "with integer division and would silently drop the ragged tail group",
                   what.c_str(), s.cols, s.group_size);
    }
    return ok();
}

/// `Q4MlxBank::validate` for a row-major bank (src/nn.rs:3348-3385).
inline Result q4_bank_validate(const TesslQ4MlxBank &bank, const TesslQuantShape &s, const std::string &what)
{
    Result r = quant_shape_validate(s, what);
    if (!r.empty()) return r;
    if (s.group_size % 32 != 0 || 512 % s.group_size != 0) {
        return fmt("%s: group_size %u is outside the MLX kernel domain {32, 64, 128, 256, 512}; the row kernels "
                   "peel each group through 16-byte loads and the simdgroup kernels stride their scale pointer "
                   "by 512 / group_size",
                   what.c_str(), s.group_size);
    }
    const uint64_t groups = elems(s.rows, s.cols / s.group_size);
    const uint64_t weights = elems(s.rows, s.cols);
    r = require(bank.packed, (weights + 1) / 2, 1, what + " packed");
    if (!r.empty()) return r;
    return require(bank.scales_biases, groups, 4, what + " scales_biases (bfloat2 per group)");
}

/// The kernels read packed rows and activations with 16-byte loads; CUDA
/// allocations are 256-byte aligned, so only a caller-made sub-view can trip this.
inline Result require_aligned16(const TesslBuf &b, const std::string &what)
{
    if (((uintptr_t)b.ptr & 15u) != 0) return fmt("%s: device pointer must be 16-byte aligned", what.c_str());
    return ok();
}

inline Result refuse_layout(uint32_t layout, const char *entry, bool takes_staged = false)
{
    if (layout == TESSL_Q4_ROW_MAJOR) return ok();
    if (layout == TESSL_Q4_B200_STAGED) {
        if (takes_staged) return ok();
        return fmt("%s: the B200 staged layout is taken by the one-row GEMV and gate/up entries only; pass a row-major bank",
                   entry);
    }
    if (layout == TESSL_Q4_INTERLEAVED4)
        return fmt("%s: the Interleaved4 layout is an Apple-GPU repack that this library does not build; "
                   "pass row-major banks", entry);
    return fmt("%s: unknown layout %u", entry, layout);
}

/// `gemm::require_i32_extent` (src/gemm.rs:34-39).
inline Result require_i32_extent(uint64_t numel, const char *what)
{
    if (numel > 0x7fffffffull) return fmt("%s exceeds signed 32-bit kernel indexing", what);
    return ok();
}

// Bound of every wait for a peer GPU: ~0.5 s of SM clocks. The peers reach the same call within
// microseconds when they run the same stream of work; a rank this late is treated as lost and the
// runtime is poisoned. tessl_runtime_set_peer_wait_limit overrides it per runtime.
constexpr long long kPeerWaitClocks = 1000000000ll;

inline Result peer_gather_validate(const TesslPeerGather &g, const char *what)
{
    if (g.world < 1 || g.world > 8) return fmt("%s: world %u is outside 1..8", what, g.world);
    if (g.rank >= g.world) return fmt("%s: rank %u is outside world %u", what, g.rank, g.world);
    if (g.bytes_per_rank % 16 != 0)
        return fmt("%s: bytes_per_rank %llu is not a multiple of 16", what, (unsigned long long)g.bytes_per_rank);
    for (uint32_t r = 0; r < g.world; ++r) {
        if (!g.buffers[r] || !g.flags[r]) return fmt("%s: rank %u has a null buffer or flag pointer", what, r);
        if (((uintptr_t)g.buffers[r] & 15u) != 0) return fmt("%s: rank %u's buffer is not 16-byte aligned", what, r);
    }
    return ok();
}

#define TESSL_TRY(expr)                   \
    do {                                  \
        ::tessl::Result _r = (expr);      \
        if (!_r.empty()) return _r;       \
    } while (0)

// ----------------------------------------------------- operator prototypes ---
// The host-side mirror of the reference's `nn::*` functions: validate, then
// launch on rt->stream. They only enqueue; waiting is the C ABI layer's job.
namespace nn {

enum OutKind : int { OUT_F32 = 0, OUT_BF16 = 1 };

Result gemv_q4_mlx_simd(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                        const TesslQuantShape &shape, uint32_t layout, const TesslBuf *resid, OutKind out);
Result gemv_q4_mlx_gate_up(TesslRuntime *rt, const char *entry, const char *what, bool silu,
                           const TesslQ4MlxBank &gate, const TesslQ4MlxBank &up, const TesslBuf &x,
                           const TesslBuf &mid, const TesslQuantShape &shape, uint32_t layout, bool mid_as_bf16);
Result gemv_q4_mlx_kv(TesslRuntime *rt, const TesslQ4MlxBank &k, const TesslQ4MlxBank &v, const TesslBuf &x_bf16,
                      const TesslBuf &k_out, const TesslBuf &v_out, const TesslQuantShape &shape, uint32_t layout);
Result gemv_q4_mlx_qkv(TesslRuntime *rt, const TesslQ4MlxBank &q, const TesslQ4MlxBank &k, const TesslQ4MlxBank &v,
                       const TesslBuf &x_bf16, const TesslQkvOutputs &out, uint32_t rows_q, uint32_t rows_kv,
                       uint32_t cols, uint32_t group_size, uint32_t layout);
Result swiglu(TesslRuntime *rt, const TesslBuf &gate, const TesslBuf &up, const TesslBuf &out, uint32_t n,
              bool out_as_bf16);
Result gemm_q4_mlx(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                   const TesslQuantShape &shape, uint32_t m, uint32_t layout, const TesslBuf *resid, OutKind out);
uint32_t gemm_q4_mlx_tensorops_max_k(uint32_t m, uint32_t n, uint32_t group_size);
Result gemm_q4_mlx_tensorops(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16,
                             const TesslBuf &y, const TesslQuantShape &shape, uint32_t m, OutKind out);
Result peer_gather(TesslRuntime *rt, const TesslPeerGather &gather);
Result gemv_q4_mlx_simd_sharded(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16,
                                const TesslPeerGather &gather, const TesslQuantShape &shape, bool y_as_bf16, bool defer = false);
Result gemv_q4_mlx_gate_up_silu_sharded(TesslRuntime *rt, const TesslQ4MlxBank &gate, const TesslQ4MlxBank &up,
                                        const TesslBuf &x_bf16, const TesslPeerGather &gather, const TesslQuantShape &shape,
                                        bool mid_as_bf16, bool defer = false);
Result peer_wait(TesslRuntime *rt, const TesslPeerGather &gather);
Result gemv_q4_mlx_simd_gathered(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslPeerGather &gather, const TesslBuf &y,
                                 const TesslQuantShape &shape, const TesslBuf *resid, OutKind out);
Result prefill_as_small_batches(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16, const TesslBuf &y,
                                const TesslQuantShape &shape, uint32_t m, OutKind out, bool *handled);
Result q8_mlx_mma(TesslRuntime *rt, const TesslBuf &codes, const TesslBuf &sb, const TesslBuf &x_bf16, const TesslBuf &y,
                  uint32_t rows, uint32_t cols, uint32_t group_size, uint32_t m, OutKind out, bool *handled);
Result gemm_q4_mlx_tensorops_noalloc(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &x_bf16,
                                     const TesslBuf &y, const TesslQuantShape &shape, uint32_t m, OutKind out);
Result gemv_q8(TesslRuntime *rt, const TesslBuf &packed, const TesslBuf &scales, const TesslBuf &zeros,
               const TesslBuf &x, const TesslBuf &y, uint32_t rows, uint32_t cols, uint32_t group_size);
Result gemm_q8_mlx(TesslRuntime *rt, const TesslBuf &codes, const TesslBuf &sb, const TesslBuf &x_bf16,
                   const TesslBuf &y, const TesslQuantShape &shape, uint32_t m, OutKind out);
Result qwen35_rms_norm(TesslRuntime *rt, const TesslBuf &x, const TesslBuf &w, const TesslBuf &out, bool out_as_bf16,
                       uint32_t rows, uint32_t dim, float eps);
Result qwen35_residual_add(TesslRuntime *rt, const TesslBuf &y, const TesslBuf &resid, uint32_t rows, uint32_t width);
Result qwen35_add_rms_norm(TesslRuntime *rt, const TesslBuf &y, const TesslBuf &resid, const TesslBuf &w, const TesslBuf &out,
                           bool out_as_bf16, uint32_t rows, uint32_t dim, float eps);
Result embed_lookup_q4_mlx(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslBuf &token_ids, const TesslBuf &out,
                           uint32_t vocab, uint32_t hidden, uint32_t group_size, uint32_t n_tokens);
uint64_t q4_mlx_staged_bytes(uint32_t rows, uint32_t cols, uint32_t group_size);
Result q4_mlx_repack_staged(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslQuantShape &shape, const TesslBuf &out);
Result q4_mlx_unpack(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslQuantShape &shape, const TesslBuf &out);
Result q4_mlx_dequant(TesslRuntime *rt, const TesslQ4MlxBank &bank, const TesslQuantShape &shape,
                      const TesslBuf &out);

}  // namespace nn

/// `Q4Weight::{matmul, gate_up_silu}` (src/qwen35_q4.rs:518-611).
namespace q4_weight {
Result matmul(TesslRuntime *rt, const TesslQ4MlxBank &bank, uint32_t rows, uint32_t cols, const TesslBuf &x_bf16,
              uint32_t m, const TesslBuf &y, const TesslBuf *resid);
Result gate_up_silu(TesslRuntime *rt, const TesslQ4MlxBank &gate, const TesslQ4MlxBank &up, uint32_t rows,
                    uint32_t cols, const TesslBuf &x_bf16, const TesslBuf &mid, bool mid_as_bf16);
}  // namespace q4_weight

}  // namespace tessl
