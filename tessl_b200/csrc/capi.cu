// The C ABI: handle ownership, status codes, the error buffer and the
// wait-before-return rule, in the conventions of the reference's src/capi.rs
// (`refuse_unowned`, `guarded`, `write_err`, `free_handle`; lines 634-774 of
// that file in the reference project). Operators are forwarded to the
// `tessl::nn` / `tessl::q4_weight` host functions.
#include <cstring>
#include <exception>
#include <new>

#include "runtime.h"

using tessl::Result;

namespace {

/// Copy `msg` NUL-terminated into `err`, truncated at a UTF-8 boundary.
void write_err(char *err, size_t err_len, const std::string &msg)
{
    if (!err || err_len == 0) return;
    size_t end = msg.size() < err_len - 1 ? msg.size() : err_len - 1;
    while (end > 0 && end < msg.size() && (static_cast<unsigned char>(msg[end]) & 0xC0) == 0x80) --end;
    std::memcpy(err, msg.data(), end);
    err[end] = 0;
}

/// Null and foreign-thread handles are refused before the handle is used.
bool refuse_unowned(TesslRuntime *rt, char *err, size_t err_len)
{
    if (!rt) {
        write_err(err, err_len, "null runtime handle");
        return true;
    }
    if (std::this_thread::get_id() != rt->owner) {
        write_err(err, err_len, "tessl runtime used from a thread other than the one that created it");
        return true;
    }
    return false;
}

Result wait_idle(TesslRuntime *rt)
{
    Result r = tessl::cuda_check(rt, cudaStreamSynchronize(rt->stream), "synchronize");
    if (!r.empty()) return r;
    if (rt->status_host && *rt->status_host != 0) {
        const uint32_t code = *rt->status_host;
        rt->poisoned = true;
        return tessl::fmt("a kernel gave up a bounded wait (status %#x: role %u, tile/step %u); its output is "
                          "incomplete and the runtime is poisoned",
                          code, code >> 24, code & 0xffffffu);
    }
    return tessl::ok();
}

/// Run `f` with every failure turned into a status. Unless encode-only mode is
/// on, the runtime is idle on return, after a success and after a failure alike
/// (a failed call may already have launched kernels that use the caller's
/// buffers); a poisoned runtime refuses new work and is not waited on.
template <typename F>
int32_t guarded(TesslRuntime *rt, char *err, size_t err_len, bool waits, F f)
{
    if (refuse_unowned(rt, err, err_len)) return TESSL_ERR;
    if (rt->poisoned) {
        write_err(err, err_len, "the runtime is poisoned by an earlier GPU fault and must be recreated");
        return TESSL_ERR;
    }
    int32_t status = TESSL_OK;
    std::string msg;
    try {
        cudaSetDevice(rt->device);
        msg = f();
        if (!msg.empty()) status = TESSL_ERR;
    } catch (const std::exception &e) {
        status = TESSL_PANIC;
        msg = std::string("panic in tessl: ") + e.what();
    } catch (...) {
        status = TESSL_PANIC;
        msg = "panic in tessl: unknown exception";
    }
    if (waits && !rt->encode_only && !rt->poisoned) {
        Result w = wait_idle(rt);
        if (!w.empty()) {
            if (status == TESSL_OK) {
                status = TESSL_ERR;
                msg = w;
            } else {
                msg += "; the wait for work already submitted then failed: " + w;
            }
        }
    }
    if (status != TESSL_OK) write_err(err, err_len, msg);
    return status;
}

TesslRuntime *make_runtime(int device, bool use_current, char *err, size_t err_len)
{
    try {
        if (use_current) {
            cudaError_t e = cudaGetDevice(&device);
            if (e != cudaSuccess) {
                write_err(err, err_len, tessl::fmt("tessl_runtime_new: no CUDA device (%s)", cudaGetErrorString(e)));
                return nullptr;
            }
        }
        cudaError_t e = cudaSetDevice(device);
        if (e != cudaSuccess) {
            write_err(err, err_len,
                      tessl::fmt("tessl_runtime_new: cannot select device %d (%s)", device, cudaGetErrorString(e)));
            return nullptr;
        }
        cudaDeviceProp prop{};
        e = cudaGetDeviceProperties(&prop, device);
        if (e != cudaSuccess) {
            write_err(err, err_len, tessl::fmt("tessl_runtime_new: %s", cudaGetErrorString(e)));
            return nullptr;
        }
        if (prop.major != 10) {
            write_err(err, err_len,
                      tessl::fmt("tessl_runtime_new: device %d is sm_%d%d; this library holds sm_100a code only",
                                 device, prop.major, prop.minor));
            return nullptr;
        }
        TesslRuntime *rt = new TesslRuntime();
        rt->device = device;
        rt->owner = std::this_thread::get_id();
        rt->sm_count = prop.multiProcessorCount;
        e = cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            write_err(err, err_len, tessl::fmt("tessl_runtime_new: cannot create a stream (%s)", cudaGetErrorString(e)));
            delete rt;
            return nullptr;
        }
        void *host = nullptr;
        e = cudaHostAlloc(&host, 64, cudaHostAllocMapped);
        if (e == cudaSuccess) e = cudaHostGetDevicePointer((void **)&rt->status_dev, host, 0);
        if (e != cudaSuccess) {
            write_err(err, err_len, tessl::fmt("tessl_runtime_new: cannot map the status word (%s)", cudaGetErrorString(e)));
            if (host) cudaFreeHost(host);
            cudaStreamDestroy(rt->stream);
            delete rt;
            return nullptr;
        }
        std::memset(host, 0, 64);
        rt->status_host = static_cast<volatile uint32_t *>(host);
        return rt;
    } catch (...) {
        write_err(err, err_len, "panic while creating the runtime");
        return nullptr;
    }
}

const TesslBuf kNoBuf{nullptr, 0};

}  // namespace

extern "C" {

uint32_t tessl_abi_version(void) { return TESSL_B200_ABI_VERSION; }

TesslRuntime *tessl_runtime_new(char *err, size_t err_len) { return make_runtime(0, true, err, err_len); }

TesslRuntime *tessl_runtime_new_on_device(int32_t device, char *err, size_t err_len)
{
    return make_runtime(device, false, err, err_len);
}

int32_t tessl_runtime_free(TesslRuntime *rt)
{
    if (!rt) return TESSL_OK;
    if (std::this_thread::get_id() != rt->owner) return TESSL_ERR;  // leaked, not freed
    cudaSetDevice(rt->device);
    if (!rt->poisoned) cudaStreamSynchronize(rt->stream);
    if (rt->scratch) cudaFree(rt->scratch);
    if (rt->status_host) cudaFreeHost((void *)rt->status_host);
    if (rt->stream) cudaStreamDestroy(rt->stream);
    delete rt;
    return TESSL_OK;
}

int32_t tessl_synchronize(TesslRuntime *rt, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, false, [&] { return wait_idle(rt); });
}

int32_t tessl_runtime_set_async_encode(TesslRuntime *rt, uint32_t on, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> Result {
        if (on > 1) return tessl::fmt("tessl_runtime_set_async_encode: on is %u, expected 0 or 1", on);
        rt->async_encode = on == 1;
        return tessl::ok();
    });
}

int32_t tessl_runtime_set_encode_only(TesslRuntime *rt, uint32_t on, char *err, size_t err_len)
{
    if (refuse_unowned(rt, err, err_len)) return TESSL_ERR;
    if (on > 1) {
        write_err(err, err_len, tessl::fmt("tessl_runtime_set_encode_only: on is %u, expected 0 or 1", on));
        return TESSL_ERR;
    }
    // Leaving the mode waits for everything enqueued under it.
    if (rt->encode_only && on == 0 && !rt->poisoned) {
        Result w = wait_idle(rt);
        if (!w.empty()) {
            write_err(err, err_len, w);
            rt->encode_only = false;
            return TESSL_ERR;
        }
    }
    rt->encode_only = on == 1;
    return TESSL_OK;
}

int32_t tessl_runtime_poisoned(TesslRuntime *rt, int32_t *out, char *err, size_t err_len)
{
    if (refuse_unowned(rt, err, err_len)) return TESSL_ERR;
    if (!out) {
        write_err(err, err_len, "tessl_runtime_poisoned: null out");
        return TESSL_ERR;
    }
    *out = rt->poisoned ? 1 : 0;
    return TESSL_OK;
}

int32_t tessl_runtime_take_dispatch_count(TesslRuntime *rt, uint64_t *out, char *err, size_t err_len)
{
    if (refuse_unowned(rt, err, err_len)) return TESSL_ERR;
    if (!out) {
        write_err(err, err_len, "tessl_runtime_take_dispatch_count: null out");
        return TESSL_ERR;
    }
    *out = rt->dispatch_count;
    rt->dispatch_count = 0;
    return TESSL_OK;
}

void *tessl_runtime_stream(TesslRuntime *rt) { return rt ? (void *)rt->stream : nullptr; }

int32_t tessl_runtime_device(TesslRuntime *rt) { return rt ? rt->device : -1; }

int32_t tessl_runtime_poison_for_test(TesslRuntime *rt)
{
    if (!rt || std::this_thread::get_id() != rt->owner) return TESSL_ERR;
    rt->poisoned = true;
    return TESSL_OK;
}

int32_t tessl_runtime_set_prefill_tile(TesslRuntime *rt, uint32_t tile_n, int32_t pair, char *err, size_t err_len)
{
    if (refuse_unowned(rt, err, err_len)) return TESSL_ERR;
    if ((tile_n != 0 && tile_n != 128 && tile_n != 192 && tile_n != 256) || pair < -1 || pair > 1) {
        write_err(err, err_len,
                  tessl::fmt("tessl_runtime_set_prefill_tile: tile_n %u is not one of [0, 128, 192, 256] or pair %d is "
                             "not one of [-1, 0, 1]", tile_n, pair));
        return TESSL_ERR;
    }
    rt->prefill_force_bn = (int)tile_n;
    rt->prefill_force_pair = pair;
    return TESSL_OK;
}

int32_t tessl_runtime_last_prefill_tile(TesslRuntime *rt, uint32_t *tile_n, uint32_t *pair, char *err, size_t err_len)
{
    if (refuse_unowned(rt, err, err_len)) return TESSL_ERR;
    if (!tile_n || !pair) {
        write_err(err, err_len, "tessl_runtime_last_prefill_tile: null out");
        return TESSL_ERR;
    }
    *tile_n = (uint32_t)rt->prefill_last_bn;
    *pair = (uint32_t)rt->prefill_last_pair;
    return TESSL_OK;
}

int32_t tessl_runtime_set_peer_wait_limit(TesslRuntime *rt, uint64_t clocks, char *err, size_t err_len)
{
    if (refuse_unowned(rt, err, err_len)) return TESSL_ERR;
    rt->peer_wait_clocks = clocks;
    return TESSL_OK;
}

int32_t tessl_buffer_alloc(TesslRuntime *rt, uint64_t nbytes, TesslBuf *out, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, false, [&]() -> Result {
        if (!out) return "tessl_buffer_alloc: null out";
        void *p = nullptr;
        // Like the reference's alloc_buffer, an empty request still yields a live buffer.
        cudaError_t e = cudaMalloc(&p, nbytes ? nbytes : 4);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return tessl::fmt("tessl_buffer_alloc: cannot allocate %llu bytes (%s)", (unsigned long long)nbytes,
                              cudaGetErrorString(e));
        }
        out->ptr = p;
        out->nbytes = nbytes ? nbytes : 4;
        return tessl::ok();
    });
}

int32_t tessl_buffer_free(TesslRuntime *rt, TesslBuf buf, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> Result {
        if (buf.ptr) return tessl::cuda_check(nullptr, cudaFree(buf.ptr), "tessl_buffer_free");
        return tessl::ok();
    });
}

int32_t tessl_buffer_write(TesslRuntime *rt, TesslBuf dst, uint64_t dst_offset, const void *src, uint64_t nbytes,
                           char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> Result {
        if (dst_offset > dst.nbytes || nbytes > dst.nbytes - dst_offset)
            return tessl::fmt("tessl_buffer_write: byte range %llu..%llu exceeds buffer capacity %llu",
                              (unsigned long long)dst_offset, (unsigned long long)(dst_offset + nbytes),
                              (unsigned long long)dst.nbytes);
        if (nbytes == 0) return tessl::ok();
        if (!src) return "tessl_buffer_write: null source";
        return tessl::cuda_check(rt,
                                 cudaMemcpyAsync(static_cast<char *>(dst.ptr) + dst_offset, src, nbytes,
                                                 cudaMemcpyHostToDevice, rt->stream),
                                 "tessl_buffer_write");
    });
}

int32_t tessl_buffer_read(TesslRuntime *rt, TesslBuf src, uint64_t src_offset, void *dst, uint64_t nbytes, char *err,
                          size_t err_len)
{
    // A read always waits, encode-only mode or not: the caller is about to look at the bytes.
    if (refuse_unowned(rt, err, err_len)) return TESSL_ERR;
    const bool was = rt->encode_only;
    rt->encode_only = false;
    const int32_t st = guarded(rt, err, err_len, true, [&]() -> Result {
        if (src_offset > src.nbytes || nbytes > src.nbytes - src_offset)
            return tessl::fmt("tessl_buffer_read: byte range %llu..%llu exceeds buffer capacity %llu",
                              (unsigned long long)src_offset, (unsigned long long)(src_offset + nbytes),
                              (unsigned long long)src.nbytes);
        if (nbytes == 0) return tessl::ok();
        if (!dst) return "tessl_buffer_read: null destination";
        return tessl::cuda_check(rt,
                                 cudaMemcpyAsync(dst, static_cast<const char *>(src.ptr) + src_offset, nbytes,
                                                 cudaMemcpyDeviceToHost, rt->stream),
                                 "tessl_buffer_read");
    });
    rt->encode_only = was;
    return st;
}

uint64_t tessl_simd_gemv_threadgroups(uint32_t rows) { return ((uint64_t)rows + 7) / 8; }

int32_t tessl_gemv_q4_mlx_simd(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y,
                               TesslQuantShape shape, uint32_t layout, const TesslBuf *resid, char *err,
                               size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemv_q4_mlx_simd(rt, bank, x_bf16, y, shape, layout, resid, tessl::nn::OUT_F32);
    });
}

int32_t tessl_gemv_q4_mlx_simd_bf16(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y_bf16,
                                    TesslQuantShape shape, uint32_t layout, const TesslBuf *resid, char *err,
                                    size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemv_q4_mlx_simd(rt, bank, x_bf16, y_bf16, shape, layout, resid, tessl::nn::OUT_BF16);
    });
}

int32_t tessl_gemv_q4_mlx_gate_up_silu(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up, TesslBuf x_bf16,
                                       TesslBuf mid, TesslQuantShape shape, uint32_t mid_as_bf16, char *err,
                                       size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemv_q4_mlx_gate_up(rt, "gemv_q4_mlx_simd_gate_up_silu", "gemv_q4_mlx_gate_up_silu", true,
                                              gate, up, x_bf16, mid, shape, TESSL_Q4_ROW_MAJOR, mid_as_bf16 != 0);
    });
}

int32_t tessl_gemv_q4_mlx_gate_up_gelu(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up, TesslBuf x_bf16,
                                       TesslBuf mid, TesslQuantShape shape, uint32_t layout, uint32_t mid_as_bf16,
                                       char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemv_q4_mlx_gate_up(rt, "gemv_q4_mlx_simd_gate_up_gelu", "gemv_q4_mlx_gate_up_gelu", false,
                                              gate, up, x_bf16, mid, shape, layout, mid_as_bf16 != 0);
    });
}

int32_t tessl_gemv_q4_mlx_kv(TesslRuntime *rt, TesslQ4MlxBank k, TesslQ4MlxBank v, TesslBuf x_bf16, TesslBuf k_out,
                             TesslBuf v_out, TesslQuantShape shape, uint32_t layout, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true,
                   [&] { return tessl::nn::gemv_q4_mlx_kv(rt, k, v, x_bf16, k_out, v_out, shape, layout); });
}

int32_t tessl_gemv_q4_mlx_qkv(TesslRuntime *rt, TesslQ4MlxBank q, TesslQ4MlxBank k, TesslQ4MlxBank v,
                              TesslBuf x_bf16, TesslQkvOutputs out, uint32_t rows_q, uint32_t rows_kv, uint32_t cols,
                              uint32_t group_size, uint32_t layout, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemv_q4_mlx_qkv(rt, q, k, v, x_bf16, out, rows_q, rows_kv, cols, group_size, layout);
    });
}

int32_t tessl_swiglu(TesslRuntime *rt, TesslBuf gate, TesslBuf up, TesslBuf out, uint32_t n, uint32_t out_as_bf16,
                     char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true,
                   [&] { return tessl::nn::swiglu(rt, gate, up, out, n, out_as_bf16 != 0); });
}

int32_t tessl_gemm_q4_mlx(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y, TesslQuantShape shape,
                          uint32_t m, uint32_t layout, const TesslBuf *resid, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemm_q4_mlx(rt, bank, x_bf16, y, shape, m, layout, resid, tessl::nn::OUT_F32);
    });
}

int32_t tessl_gemm_q4_mlx_bf16(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y_bf16,
                               TesslQuantShape shape, uint32_t m, uint32_t layout, const TesslBuf *resid, char *err,
                               size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemm_q4_mlx(rt, bank, x_bf16, y_bf16, shape, m, layout, resid, tessl::nn::OUT_BF16);
    });
}

uint32_t tessl_gemm_q4_mlx_tensorops_max_k(uint32_t m, uint32_t n, uint32_t group_size)
{
    return tessl::nn::gemm_q4_mlx_tensorops_max_k(m, n, group_size);
}

int32_t tessl_gemm_q4_mlx_tensorops(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y,
                                    TesslQuantShape shape, uint32_t m, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemm_q4_mlx_tensorops(rt, bank, x_bf16, y, shape, m, tessl::nn::OUT_F32);
    });
}

int32_t tessl_gemm_q4_mlx_tensorops_bf16(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y_bf16,
                                         TesslQuantShape shape, uint32_t m, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemm_q4_mlx_tensorops(rt, bank, x_bf16, y_bf16, shape, m, tessl::nn::OUT_BF16);
    });
}

int32_t tessl_gemm_q4_mlx_tensorops_noalloc(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y,
                                            TesslQuantShape shape, uint32_t m, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemm_q4_mlx_tensorops_noalloc(rt, bank, x_bf16, y, shape, m, tessl::nn::OUT_F32);
    });
}

int32_t tessl_peer_gather(TesslRuntime *rt, const TesslPeerGather *gather, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> tessl::Result {
        if (!gather) return "peer_gather: null descriptor";
        return tessl::nn::peer_gather(rt, *gather);
    });
}

int32_t tessl_gemv_q4_mlx_simd_sharded(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, const TesslPeerGather *gather,
                                       TesslQuantShape shape, uint32_t y_as_bf16, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> tessl::Result {
        if (!gather) return "gemv_q4_mlx_simd_sharded: null descriptor";
        return tessl::nn::gemv_q4_mlx_simd_sharded(rt, bank, x_bf16, *gather, shape, y_as_bf16 != 0);
    });
}

int32_t tessl_gemv_q4_mlx_simd_sharded_deferred(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16,
                                                const TesslPeerGather *gather, TesslQuantShape shape, uint32_t y_as_bf16,
                                                char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> tessl::Result {
        if (!gather) return "gemv_q4_mlx_simd_sharded_deferred: null descriptor";
        return tessl::nn::gemv_q4_mlx_simd_sharded(rt, bank, x_bf16, *gather, shape, y_as_bf16 != 0, true);
    });
}

int32_t tessl_gemv_q4_mlx_gate_up_silu_sharded_deferred(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up,
                                                        TesslBuf x_bf16, const TesslPeerGather *gather, TesslQuantShape shape,
                                                        uint32_t mid_as_bf16, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> tessl::Result {
        if (!gather) return "gemv_q4_mlx_gate_up_silu_sharded_deferred: null descriptor";
        return tessl::nn::gemv_q4_mlx_gate_up_silu_sharded(rt, gate, up, x_bf16, *gather, shape, mid_as_bf16 != 0, true);
    });
}

int32_t tessl_gemv_q4_mlx_simd_gathered(TesslRuntime *rt, TesslQ4MlxBank bank, const TesslPeerGather *gather, TesslBuf y,
                                        TesslQuantShape shape, const TesslBuf *resid, uint32_t y_as_bf16, char *err,
                                        size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> tessl::Result {
        if (!gather) return "gemv_q4_mlx_simd_gathered: null descriptor";
        return tessl::nn::gemv_q4_mlx_simd_gathered(rt, bank, *gather, y, shape, resid,
                                                    y_as_bf16 ? tessl::nn::OUT_BF16 : tessl::nn::OUT_F32);
    });
}

int32_t tessl_peer_wait(TesslRuntime *rt, const TesslPeerGather *gather, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> tessl::Result {
        if (!gather) return "peer_wait: null descriptor";
        return tessl::nn::peer_wait(rt, *gather);
    });
}

int32_t tessl_gemv_q4_mlx_gate_up_silu_sharded(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up, TesslBuf x_bf16,
                                               const TesslPeerGather *gather, TesslQuantShape shape, uint32_t mid_as_bf16,
                                               char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&]() -> tessl::Result {
        if (!gather) return "gemv_q4_mlx_gate_up_silu_sharded: null descriptor";
        return tessl::nn::gemv_q4_mlx_gate_up_silu_sharded(rt, gate, up, x_bf16, *gather, shape, mid_as_bf16 != 0);
    });
}

uint64_t tessl_q4_mlx_staged_bytes(uint32_t rows, uint32_t cols, uint32_t group_size)
{
    return tessl::nn::q4_mlx_staged_bytes(rows, cols, group_size);
}

int32_t tessl_q4_mlx_repack_staged(TesslRuntime *rt, TesslQ4MlxBank bank, TesslQuantShape shape, TesslBuf out, char *err,
                                   size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] { return tessl::nn::q4_mlx_repack_staged(rt, bank, shape, out); });
}

int32_t tessl_gemv_q4_mlx_gate_up_silu_layout(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up, TesslBuf x_bf16,
                                              TesslBuf mid, TesslQuantShape shape, uint32_t layout, uint32_t mid_as_bf16,
                                              char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemv_q4_mlx_gate_up(rt, "gemv_q4_mlx_simd_gate_up_silu", "gemv_q4_mlx_gate_up_silu", true, gate,
                                              up, x_bf16, mid, shape, layout, mid_as_bf16 != 0);
    });
}

int32_t tessl_q4_weight_matmul(TesslRuntime *rt, TesslQ4MlxBank bank, uint32_t rows, uint32_t cols, TesslBuf x_bf16,
                               uint32_t m, TesslBuf y, const TesslBuf *resid, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true,
                   [&] { return tessl::q4_weight::matmul(rt, bank, rows, cols, x_bf16, m, y, resid); });
}

int32_t tessl_q4_weight_gate_up_silu(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up, uint32_t rows,
                                     uint32_t cols, TesslBuf x_bf16, TesslBuf mid, uint32_t mid_as_bf16, char *err,
                                     size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::q4_weight::gate_up_silu(rt, gate, up, rows, cols, x_bf16, mid, mid_as_bf16 != 0);
    });
}

int32_t tessl_gemv_q8(TesslRuntime *rt, TesslBuf packed, TesslBuf scales, TesslBuf zeros, TesslBuf x, TesslBuf y,
                      uint32_t rows, uint32_t cols, uint32_t group_size, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true,
                   [&] { return tessl::nn::gemv_q8(rt, packed, scales, zeros, x, y, rows, cols, group_size); });
}

int32_t tessl_gemm_q8_mlx(TesslRuntime *rt, TesslBuf codes, TesslBuf scales_biases, TesslBuf x_bf16, TesslBuf y,
                          TesslQuantShape shape, uint32_t m, uint32_t y_as_bf16, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::gemm_q8_mlx(rt, codes, scales_biases, x_bf16, y, shape, m,
                                      y_as_bf16 ? tessl::nn::OUT_BF16 : tessl::nn::OUT_F32);
    });
}

int32_t tessl_embed_lookup_q4_mlx(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf token_ids, TesslBuf out, uint32_t vocab,
                                  uint32_t hidden, uint32_t group_size, uint32_t n_tokens, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::embed_lookup_q4_mlx(rt, bank, token_ids, out, vocab, hidden, group_size, n_tokens);
    });
}

int32_t tessl_qwen35_rms_norm(TesslRuntime *rt, TesslBuf x, TesslBuf w, TesslBuf out, uint32_t out_as_bf16, uint32_t rows,
                              uint32_t dim, float eps, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true,
                   [&] { return tessl::nn::qwen35_rms_norm(rt, x, w, out, out_as_bf16 != 0, rows, dim, eps); });
}

int32_t tessl_qwen35_residual_add(TesslRuntime *rt, TesslBuf y, TesslBuf resid, uint32_t rows, uint32_t width, char *err,
                                  size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] { return tessl::nn::qwen35_residual_add(rt, y, resid, rows, width); });
}

int32_t tessl_qwen35_add_rms_norm(TesslRuntime *rt, TesslBuf y, TesslBuf resid, TesslBuf w, TesslBuf out,
                                  uint32_t out_as_bf16, uint32_t rows, uint32_t dim, float eps, char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] {
        return tessl::nn::qwen35_add_rms_norm(rt, y, resid, w, out, out_as_bf16 != 0, rows, dim, eps);
    });
}

int32_t tessl_q4_mlx_unpack(TesslRuntime *rt, TesslQ4MlxBank bank, TesslQuantShape shape, TesslBuf out_u8, char *err,
                            size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] { return tessl::nn::q4_mlx_unpack(rt, bank, shape, out_u8); });
}

int32_t tessl_q4_mlx_dequant(TesslRuntime *rt, TesslQ4MlxBank bank, TesslQuantShape shape, TesslBuf out_f32,
                             char *err, size_t err_len)
{
    return guarded(rt, err, err_len, true, [&] { return tessl::nn::q4_mlx_dequant(rt, bank, shape, out_f32); });
}

}  // extern "C"
