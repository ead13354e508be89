/* tessl_b200: the MLX affine-quantized matmul path of bharathvbcr/tessl for NVIDIA B200.
 *
 * A C ABI in the conventions of the reference's `src/capi.rs`: an opaque,
 * thread-affine runtime handle, an `int32_t` status with the message written
 * NUL-terminated into a caller buffer (`err` may be NULL), every argument
 * validated before any GPU work, and each call returning with the runtime
 * idle unless encode-only mode is on.
 *
 * Each operator entry below replaces one function of the reference's typed
 * kernel API (`src/nn.rs`, `src/qwen35_q4.rs`); the citation names the file
 * and lines of the reference project it mirrors. Argument order follows the
 * Rust signature. A `GpuBuffer` becomes a `TesslBuf`: a device pointer plus
 * its capacity in bytes, which the library checks against what a kernel will
 * read or write exactly as `nn::require` does (src/nn.rs:126-143).
 */
#ifndef TESSL_B200_H
#define TESSL_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TESSL_API __attribute__((visibility("default")))
#else
#define TESSL_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes (src/capi.rs:78-80). */
#define TESSL_OK 0
#define TESSL_ERR 1
#define TESSL_PANIC 2

/* Bumped on any change to a struct layout or a signature below; bindings
 * refuse a library whose version differs (src/capi.rs:82-91). */
#define TESSL_B200_ABI_VERSION 1u

/* Largest M of the small-batch kernel (src/nn.rs:4524). */
#define TESSL_GEMM_Q4_MLX_MAX_M 8u

typedef struct TesslRuntime TesslRuntime;

/* Device memory handed to an operator: pointer and capacity in bytes. */
typedef struct TesslBuf {
    void *ptr;
    uint64_t nbytes;
} TesslBuf;

/* src/nn.rs:3238-3245. */
typedef struct TesslQuantShape {
    uint32_t rows;       /* output rows N */
    uint32_t cols;       /* reduction length K */
    uint32_t group_size; /* weights per (scale, bias) pair; must divide cols */
} TesslQuantShape;

/* src/nn.rs:3332-3338: packed nibbles (two per byte, low first = MLX's
 * little-endian U32 words) and one bf16 (scale, bias) pair per group. */
typedef struct TesslQ4MlxBank {
    TesslBuf packed;
    TesslBuf scales_biases;
} TesslQ4MlxBank;

/* src/nn.rs:3669-3675. Of the reference's two layouts the row-major one is built;
 * Interleaved4 (an Apple-GPU repack no Qwen3.5 path uses) is refused by name. */
#define TESSL_Q4_ROW_MAJOR 0u
#define TESSL_Q4_INTERLEAVED4 1u
/* An offline repack for this library's GEMV kernel (the role Interleaved4 plays on
 * Apple GPUs; no counterpart in the reference): see tessl_q4_mlx_repack_staged. */
#define TESSL_Q4_B200_STAGED 2u

/* src/nn.rs:4408-4415. */
typedef struct TesslQkvOutputs {
    TesslBuf q_out;
    TesslBuf k_out;
    TesslBuf v_out;
} TesslQkvOutputs;

/* ------------------------------------------------------------- runtime --- */

/* src/capi.rs:186-189. */
TESSL_API uint32_t tessl_abi_version(void);

/* A runtime on the calling thread's current CUDA device, with a stream of its
 * own; NULL with the reason in `err` on failure (src/capi.rs:255-276). */
TESSL_API TesslRuntime *tessl_runtime_new(char *err, size_t err_len);

/* The same on a named device ordinal. No counterpart in the reference, which
 * has one system default device; multi-GPU hosts need to choose. */
TESSL_API TesslRuntime *tessl_runtime_new_on_device(int32_t device, char *err, size_t err_len);

/* Free on the creating thread; NULL is ignored; a foreign thread leaks the
 * handle and gets TESSL_ERR (src/capi.rs:278-293). */
TESSL_API int32_t tessl_runtime_free(TesslRuntime *rt);

/* Wait for all submitted work (src/capi.rs:295-303). */
TESSL_API int32_t tessl_synchronize(TesslRuntime *rt, char *err, size_t err_len);

/* Accepted for signature compatibility (src/capi.rs:305-332): `on` must be 0
 * or 1. Every call here is already a single submission that is waited for once,
 * which is what the reference's async-encode mode gives; the mode changes
 * nothing a caller can observe. */
TESSL_API int32_t tessl_runtime_set_async_encode(TesslRuntime *rt, uint32_t on, char *err, size_t err_len);

/* Encode-only mode: operators enqueue their kernels on the runtime's stream
 * and return without waiting, the contract of the Rust `nn::*` functions
 * themselves (src/lib.rs:96-106), for callers that batch a whole token's
 * projections and wait once with tessl_synchronize. Off by default. */
TESSL_API int32_t tessl_runtime_set_encode_only(TesslRuntime *rt, uint32_t on, char *err, size_t err_len);

/* 1 when a CUDA fault has latched the runtime (every later call is refused),
 * else 0; works on a poisoned runtime (src/capi.rs:212-247). */
TESSL_API int32_t tessl_runtime_poisoned(TesslRuntime *rt, int32_t *out, char *err, size_t err_len);

/* Kernels launched since the last call, then reset to zero: lets a caller
 * prove a refused call did no GPU work (`take_dispatch_count`,
 * tests/gemm_q4_mlx_tensorops.rs:374 in the reference project). */
TESSL_API int32_t tessl_runtime_take_dispatch_count(TesslRuntime *rt, uint64_t *out, char *err, size_t err_len);

/* The runtime's CUDA stream (a `cudaStream_t`) and device ordinal, so a caller
 * can order its own work or record events around operator calls. */
TESSL_API void *tessl_runtime_stream(TesslRuntime *rt);
TESSL_API int32_t tessl_runtime_device(TesslRuntime *rt);

/* Test hook: latch the poison flag without a GPU fault (the reference's
 * `poison_as_shared_event_timeout_for_test`, src/runtime.rs:1076). */
TESSL_API int32_t tessl_runtime_poison_for_test(TesslRuntime *rt);

/* Prefill GEMM tile choice, for tuning runs and for tests that must reach every
 * compiled tile: tile_n in {128, 192, 256} forces the tile width of later
 * tessl_gemm_q4_mlx_tensorops* calls on this runtime (0 = the library's own
 * estimate), pair = 1 / 0 forces the two-CTA or the single-CTA kernel (-1 = the
 * library decides). tessl_runtime_last_prefill_tile reports what the most
 * recent prefill call launched (tile_n = 0 if it ran no tile kernel). No
 * counterpart in the reference, whose kernel has one 32 x 32 tile. */
TESSL_API int32_t tessl_runtime_set_prefill_tile(TesslRuntime *rt, uint32_t tile_n, int32_t pair, char *err, size_t err_len);
TESSL_API int32_t tessl_runtime_last_prefill_tile(TesslRuntime *rt, uint32_t *tile_n, uint32_t *pair, char *err,
                                        size_t err_len);

/* Clock budget (SM clocks) of the bounded waits a kernel of this runtime makes
 * on another GPU's flags (tessl_peer_gather and the sharded GEMV's exchange);
 * 0 restores the default of about half a second. A wait that runs out makes the
 * kernel write a status word and return; the next wait on the host reports it
 * and poisons the runtime, the way the reference reports a shared-event
 * timeout (src/runtime.rs:1498-1531). A test uses a small budget to exercise
 * that path without sitting through the default one. */
TESSL_API int32_t tessl_runtime_set_peer_wait_limit(TesslRuntime *rt, uint64_t clocks, char *err, size_t err_len);

/* Device buffers (`GpuRuntime::alloc_buffer`, `GpuBuffer::write_bytes`,
 * `read_*`; src/runtime.rs:2083, src/tensor.rs). Copies are ordered on the
 * runtime's stream and complete before return. */
TESSL_API int32_t tessl_buffer_alloc(TesslRuntime *rt, uint64_t nbytes, TesslBuf *out, char *err, size_t err_len);
TESSL_API int32_t tessl_buffer_free(TesslRuntime *rt, TesslBuf buf, char *err, size_t err_len);
TESSL_API int32_t tessl_buffer_write(TesslRuntime *rt, TesslBuf dst, uint64_t dst_offset, const void *src, uint64_t nbytes,
                           char *err, size_t err_len);
TESSL_API int32_t tessl_buffer_read(TesslRuntime *rt, TesslBuf src, uint64_t src_offset, void *dst, uint64_t nbytes,
                          char *err, size_t err_len);

/* ---------------------------------------------------------- Q4 GEMV (M=1) --- */

/* `nn::simd_gemv_threadgroups` (src/nn.rs:3699-3701): ceil(rows / 8). Kept so
 * callers that reason about the reference's grid partition still can; this
 * library sizes its own grids. */
TESSL_API uint64_t tessl_simd_gemv_threadgroups(uint32_t rows);

/* `nn::gemv_q4_mlx_simd` (src/nn.rs:3982-4074): y[rows] = W x (+ resid), x bf16
 * [cols], y f32 [rows], resid f32 [rows] or NULL; resid may be y itself. */
TESSL_API int32_t tessl_gemv_q4_mlx_simd(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y,
                               TesslQuantShape shape, uint32_t layout, const TesslBuf *resid, char *err,
                               size_t err_len);

/* The same with y stored as bf16 (round to nearest even of the f32 result).
 * No counterpart in the reference, whose GEMVs always store f32; provided for
 * callers that keep activations in bf16. resid stays f32. */
TESSL_API int32_t tessl_gemv_q4_mlx_simd_bf16(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y_bf16,
                                    TesslQuantShape shape, uint32_t layout, const TesslBuf *resid, char *err,
                                    size_t err_len);

/* `nn::gemv_q4_mlx_gate_up_silu` (src/nn.rs:4165-4194): mid[rows] =
 * silu(W_gate x) * (W_up x) in one launch; mid is bf16 when mid_as_bf16 != 0,
 * else f32. */
TESSL_API int32_t tessl_gemv_q4_mlx_gate_up_silu(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up, TesslBuf x_bf16,
                                       TesslBuf mid, TesslQuantShape shape, uint32_t mid_as_bf16, char *err,
                                       size_t err_len);

/* `nn::gemv_q4_mlx_gate_up_gelu` with `GateUpDispatch::Simd(layout)`
 * (src/nn.rs:4098-4155): the same with tanh-approximate GELU. */
TESSL_API int32_t tessl_gemv_q4_mlx_gate_up_gelu(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up, TesslBuf x_bf16,
                                       TesslBuf mid, TesslQuantShape shape, uint32_t layout, uint32_t mid_as_bf16,
                                       char *err, size_t err_len);

/* `nn::gemv_q4_mlx_kv` (src/nn.rs:4279-4351): k_out = W_k x and v_out = W_v x
 * in one launch; both banks share `shape`. */
TESSL_API int32_t tessl_gemv_q4_mlx_kv(TesslRuntime *rt, TesslQ4MlxBank k, TesslQ4MlxBank v, TesslBuf x_bf16, TesslBuf k_out,
                             TesslBuf v_out, TesslQuantShape shape, uint32_t layout, char *err, size_t err_len);

/* `nn::gemv_q4_mlx_qkv` (src/nn.rs:4366-4515): three projections of one x in
 * one launch; Q has rows_q rows, K and V rows_kv. */
TESSL_API int32_t tessl_gemv_q4_mlx_qkv(TesslRuntime *rt, TesslQ4MlxBank q, TesslQ4MlxBank k, TesslQ4MlxBank v,
                              TesslBuf x_bf16, TesslQkvOutputs out, uint32_t rows_q, uint32_t rows_kv, uint32_t cols,
                              uint32_t group_size, uint32_t layout, char *err, size_t err_len);

/* `qwen35::swiglu` as `Qwen35Model::gate_up_silu` uses it when the fused
 * kernel is off (src/qwen35_model.rs:1938-1957): out[i] = silu(gate[i]) * up[i]
 * over n f32 values, out f32 or bf16. The fused entry above is bit-identical
 * to two tessl_gemv_q4_mlx_simd calls followed by this. */
TESSL_API int32_t tessl_swiglu(TesslRuntime *rt, TesslBuf gate, TesslBuf up, TesslBuf out, uint32_t n, uint32_t out_as_bf16,
                     char *err, size_t err_len);

/* ------------------------------------------------- Q4 GEMM, small and large M --- */

/* `nn::gemm_q4_mlx` (src/nn.rs:4535-4619): Y[m, rows] = X[m, cols] W^T
 * (+ resid) for m <= 8; X bf16 row-major, Y and resid f32 [m, rows]. */
TESSL_API int32_t tessl_gemm_q4_mlx(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y, TesslQuantShape shape,
                          uint32_t m, uint32_t layout, const TesslBuf *resid, char *err, size_t err_len);

/* bf16-output twin of tessl_gemm_q4_mlx (no counterpart in the reference). */
TESSL_API int32_t tessl_gemm_q4_mlx_bf16(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y_bf16,
                               TesslQuantShape shape, uint32_t m, uint32_t layout, const TesslBuf *resid, char *err,
                               size_t err_len);

/* `nn::gemm_q4_mlx_tensorops_max_k` (src/nn.rs:4650-4655). */
TESSL_API uint32_t tessl_gemm_q4_mlx_tensorops_max_k(uint32_t m, uint32_t n, uint32_t group_size);

/* `nn::gemm_q4_mlx_tensorops` (src/nn.rs:4683-4757): the prefill GEMM for any
 * m, group_size in {32, 64, 128}, row-major bank, no residual; Y f32 [m, rows].
 * Runs on the tcgen05 tensor cores. */
TESSL_API int32_t tessl_gemm_q4_mlx_tensorops(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y,
                                    TesslQuantShape shape, uint32_t m, char *err, size_t err_len);

/* bf16-output twin of tessl_gemm_q4_mlx_tensorops (no counterpart in the reference). */
TESSL_API int32_t tessl_gemm_q4_mlx_tensorops_bf16(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y_bf16,
                                         TesslQuantShape shape, uint32_t m, char *err, size_t err_len);

/* tessl_gemm_q4_mlx_tensorops for callers that cannot allocate device memory.
 * It has no counterpart in the reference. The regular entry keeps its
 * intermediate data (an f16 copy of X with per-group sums, and one scale per
 * row) in a buffer it grows with cudaMalloc; a serving loop that forbids
 * allocation in steady state (cudaMalloc can synchronise the device and can fail
 * when memory is tight) or code living under another framework's allocator
 * cannot afford that call. This entry
 * uses a fixed 8 MiB array inside the library instead (held by every GPU that
 * loads the library until the process exits) and refuses, with a message that
 * names the sizes, any call whose m * K_aug * 2 + m * 4 bytes do not fit
 * (K_aug = 64 * (ceil(K/64) + ceil(4*(K/G)/64)); e.g. up to m = 963 at K = 4096,
 * G = 64). Arguments, validation, kernels and results are those of
 * tessl_gemm_q4_mlx_tensorops. The first call on a device looks the array's
 * address up (a synchronous query of the CUDA runtime). All calls on a device
 * share the array: it keeps the previous call's contents (every byte a call
 * reads is rewritten by that call first, so nothing needs clearing), and calls
 * that overlap on the GPU race on it - serialise them. */
TESSL_API int32_t tessl_gemm_q4_mlx_tensorops_noalloc(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16, TesslBuf y,
                                            TesslQuantShape shape, uint32_t m, char *err, size_t err_len);

/* All-gather of per-GPU output slices through NVLink peer memory: NO COUNTERPART IN
 * THE REFERENCE (a single-device library). For the column-sharded GEMVs, whose
 * outputs are too small for a library all-gather to be anything but latency.
 * `buffers[r]` is rank r's gather buffer (world * bytes_per_rank bytes, peer
 * mapped on this GPU, 16-byte aligned), `flags[r]` rank r's 18 zero-initialised
 * 32-bit flag words (peer mapped as well). Each rank writes its slice into
 * buffers[rank] + rank * bytes_per_rank (the GEMV can do that directly), then
 * every rank makes this call on its own stream; when the call's kernel has
 * finished, buffers[rank] holds all slices. Calls must be made in the same order
 * on every rank. The kernel waits for its peers with a ~0.5 s bound; on expiry the
 * runtime is poisoned. May be captured in a CUDA graph. */
typedef struct TesslPeerGather {
    void *buffers[8];
    uint32_t *flags[8];
    uint32_t rank;
    uint32_t world;
    uint64_t bytes_per_rank;
} TesslPeerGather;
TESSL_API int32_t tessl_peer_gather(TesslRuntime *rt, const TesslPeerGather *gather, char *err, size_t err_len);

/* tessl_gemv_q4_mlx_simd / tessl_gemv_q4_mlx_gate_up_silu on this rank's row slice
 * of a column-sharded bank, with the exchange inside the GEMV kernel: NO
 * COUNTERPART IN THE REFERENCE. `shape.rows` are the slice's rows; the f32 (or
 * bf16) results go to byte offset rank * bytes_per_rank of EVERY rank's gather
 * buffer - the warp that finishes an output row stores it locally and to each
 * peer with plain NVLink stores - and the launch ends with one bounded flag
 * exchange, after which buffers[rank] holds every rank's slice, as after
 * tessl_peer_gather. One launch and one exposed flag round trip instead of two
 * launches and two. Same descriptor, flag words and calling rules as
 * tessl_peer_gather (every rank makes the matching call in the same order; the
 * two kinds of call may be mixed on one descriptor); a rank whose slice is empty
 * calls tessl_peer_gather instead. Shapes the tensor-core GEMV does not take
 * (cols outside {1024, 2048, 4096}) run as the plain GEMV followed by
 * tessl_peer_gather, with the same result. */
TESSL_API int32_t tessl_gemv_q4_mlx_simd_sharded(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16,
                                       const TesslPeerGather *gather, TesslQuantShape shape, uint32_t y_as_bf16,
                                       char *err, size_t err_len);
TESSL_API int32_t tessl_gemv_q4_mlx_gate_up_silu_sharded(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up,
                                               TesslBuf x_bf16, const TesslPeerGather *gather, TesslQuantShape shape,
                                               uint32_t mid_as_bf16, char *err, size_t err_len);

/* The same two launches without the last wait: the kernel stores its outputs to
 * every rank, tells the peers that they are complete and ends; it does NOT wait
 * for the peers' slices. The reader of the gathered vector does that instead -
 * tessl_gemv_q4_mlx_simd_gathered inside its kernel, behind that kernel's own
 * weight prefetch, or tessl_peer_wait as a launch of its own before any other
 * reader - so the NVLink round trip is no longer exposed between the two
 * launches. After a deferred call, buffers[rank] must not be read by anything
 * else first. NO COUNTERPART IN THE REFERENCE. */
TESSL_API int32_t tessl_gemv_q4_mlx_simd_sharded_deferred(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf x_bf16,
                                                const TesslPeerGather *gather, TesslQuantShape shape,
                                                uint32_t y_as_bf16, char *err, size_t err_len);
TESSL_API int32_t tessl_gemv_q4_mlx_gate_up_silu_sharded_deferred(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up,
                                                        TesslBuf x_bf16, const TesslPeerGather *gather,
                                                        TesslQuantShape shape, uint32_t mid_as_bf16, char *err,
                                                        size_t err_len);
/* tessl_gemv_q4_mlx_simd[_bf16] whose x is the gathered vector buffers[rank]
 * (bf16, world * bytes_per_rank bytes) of `gather`: before reading x the kernel
 * waits, bounded like every peer wait, until every peer's completion flag has
 * reached this rank's call counter. Correct after a deferred and after a waiting
 * exchange alike. */
TESSL_API int32_t tessl_gemv_q4_mlx_simd_gathered(TesslRuntime *rt, TesslQ4MlxBank bank, const TesslPeerGather *gather,
                                        TesslBuf y, TesslQuantShape shape, const TesslBuf *resid, uint32_t y_as_bf16,
                                        char *err, size_t err_len);
/* The deferred wait as a launch of its own, for any other reader of buffers[rank]. */
TESSL_API int32_t tessl_peer_wait(TesslRuntime *rt, const TesslPeerGather *gather, char *err, size_t err_len);

/* `Q4Weight::matmul` (src/qwen35_q4.rs:518-561): the M-dispatch policy over one
 * bank of group size 64. m == 0 is a no-op, 1 the GEMV, 2..=8 the small-batch
 * kernel, more the tensor-core GEMM (which refuses a residual). x is bf16
 * [m, cols], y f32 [m, rows]. */
TESSL_API int32_t tessl_q4_weight_matmul(TesslRuntime *rt, TesslQ4MlxBank bank, uint32_t rows, uint32_t cols, TesslBuf x_bf16,
                               uint32_t m, TesslBuf y, const TesslBuf *resid, char *err, size_t err_len);

/* `Q4Weight::gate_up_silu` (src/qwen35_q4.rs:568-611): one row, group 64. */
TESSL_API int32_t tessl_q4_weight_gate_up_silu(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up, uint32_t rows,
                                     uint32_t cols, TesslBuf x_bf16, TesslBuf mid, uint32_t mid_as_bf16, char *err,
                                     size_t err_len);

/* ------------------------------------------------------------------- Q8 --- */

/* `nn::gemv_q8` (src/nn.rs:716-795): y[rows] = W x, W signed int8 row-major,
 * f32 scales and zeros per group, w = scale * (q - zero), f32 x, f32 y. */
TESSL_API int32_t tessl_gemv_q8(TesslRuntime *rt, TesslBuf packed, TesslBuf scales, TesslBuf zeros, TesslBuf x, TesslBuf y,
                      uint32_t rows, uint32_t cols, uint32_t group_size, char *err, size_t err_len);

/* MLX-layout 8-bit GEMV/GEMM for m <= 8: unsigned codes 0..255 (four per
 * little-endian U32), bf16 (scale, bias) pairs, w = scale * code + bias, X bf16
 * [m, cols]; Y f32 [m, rows], or bf16 when y_as_bf16 != 0. No counterpart in the
 * reference (its only Q8 kernel is tessl_gemv_q8's); this is the Q4 bank
 * convention at eight bits. group_size in {32, 64, 128, 256, 512}. */
TESSL_API int32_t tessl_gemm_q8_mlx(TesslRuntime *rt, TesslBuf codes, TesslBuf scales_biases, TesslBuf x_bf16, TesslBuf y,
                          TesslQuantShape shape, uint32_t m, uint32_t y_as_bf16, char *err, size_t err_len);

/* ------------------------------------------------------ embedding gather --- */

/* `nn::embed_lookup_q4_mlx` (src/nn.rs:3592-3658; kernels/embed_lookup.metal:7-38):
 * out[m, :] = the dequantized row token_ids[m] of an MLX Q4 table [vocab, hidden]
 * (w = scale * q + bias, separate multiply and add), f32 [n_tokens, hidden];
 * token_ids u32 [n_tokens]; an id >= vocab gives a row of zeros. First operator
 * of every decode step (src/qwen35_model.rs:1476). */
TESSL_API int32_t tessl_embed_lookup_q4_mlx(TesslRuntime *rt, TesslQ4MlxBank bank, TesslBuf token_ids, TesslBuf out,
                                  uint32_t vocab, uint32_t hidden, uint32_t group_size, uint32_t n_tokens, char *err,
                                  size_t err_len);

/* ------------------------------------------ either side of a projection --- */

/* `qwen35::rms_norm` (src/qwen35.rs:2654-2695; kernels/qwen35_mlp.metal:76-122):
 * out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * (1 + w[:]); x f32 [rows, dim],
 * w f32 [dim] as the checkpoint holds it, out f32 or (out_as_bf16 != 0) bf16 -
 * the activations a Q4 projection reads. An f32 out may be x itself. */
TESSL_API int32_t tessl_qwen35_rms_norm(TesslRuntime *rt, TesslBuf x, TesslBuf w, TesslBuf out, uint32_t out_as_bf16,
                              uint32_t rows, uint32_t dim, float eps, char *err, size_t err_len);

/* `qwen35::residual_add` for dense operands (src/qwen35.rs:2586-2623): resid += y,
 * f32 [rows, width]. */
TESSL_API int32_t tessl_qwen35_residual_add(TesslRuntime *rt, TesslBuf y, TesslBuf resid, uint32_t rows, uint32_t width,
                                  char *err, size_t err_len);

/* `qwen35::add_rms_norm` (src/qwen35.rs:2697-2747; kernels/qwen35_mlp.metal:124-171):
 * resid += y, then out = rms_norm(resid) * (1 + w), in one launch; bit-identical
 * to tessl_qwen35_residual_add followed by tessl_qwen35_rms_norm. */
TESSL_API int32_t tessl_qwen35_add_rms_norm(TesslRuntime *rt, TesslBuf y, TesslBuf resid, TesslBuf w, TesslBuf out,
                                  uint32_t out_as_bf16, uint32_t rows, uint32_t dim, float eps, char *err,
                                  size_t err_len);

/* ------------------------------------------------- checkpoint -> bank --- */

/* A safetensors file opened read-only (memory-mapped) with its header parsed
 * and checked: every entry's dtype, shape and data_offsets agree, the ranges
 * lie inside the file and do not overlap. Stands in for the safetensors crate
 * behind `Loader::open` (src/loader.rs:33-118). Host only; NULL + err on refusal. */
typedef struct TesslCheckpoint TesslCheckpoint;
typedef struct TesslTensorInfo {
    char dtype[8];      /* "U32", "BF16", "F32", ... as the header spells it */
    uint32_t ndim;
    uint64_t shape[8];
    uint64_t nbytes;
} TesslTensorInfo;

TESSL_API TesslCheckpoint *tessl_checkpoint_open(const char *path, char *err, size_t err_len);
TESSL_API void tessl_checkpoint_close(TesslCheckpoint *ck);
TESSL_API int32_t tessl_checkpoint_tensor_count(const TesslCheckpoint *ck, uint64_t *out, char *err, size_t err_len);
TESSL_API int32_t tessl_checkpoint_tensor_name(const TesslCheckpoint *ck, uint64_t index, char *name, size_t name_len,
                                     char *err, size_t err_len);
/* `Loader::tensor_info` (src/loader.rs:120-140): header facts, no bytes read. */
TESSL_API int32_t tessl_checkpoint_tensor_info(const TesslCheckpoint *ck, const char *name, TesslTensorInfo *out, char *err,
                                     size_t err_len);

/* `MlxQuant::from_config_json` (src/qwen35_q4.rs:204-255): the `quantization`
 * object of an mlx-lm config.json. Accepts only one uniform affine 4-bit
 * group-64 quantization; a per-layer entry, another mode, width or group, or
 * `quantization` and `quantization_config` that differ, are refused by name. */
TESSL_API int32_t tessl_mlx_quant_from_config_json(const char *text, uint32_t *bits, uint32_t *group_size, char *err,
                                         size_t err_len);

/* `MlxNames::detect` (src/qwen35_q4.rs:268-293): how a checkpoint spells its
 * tower, from its tensor names: "language_model.model." + "language_model.lm_head"
 * (mlx-lm) or "model.language_model." + "lm_head" (Hugging Face). `*prefix` and
 * `*head` point at constants of the library. Neither present, or both, is refused. */
TESSL_API int32_t tessl_mlx_names_detect(const char *const *names, uint64_t n, const char **prefix, const char **head,
                               char *err, size_t err_len);

/* `NormConvention::from_conv_shape` (src/qwen35_q4.rs:296-336): a GDN layer's
 * conv1d.weight of shape [conv_dim, 1, kernel] means the transformers layout
 * (*convention = 0: norm weights hold w), [conv_dim, kernel, 1] the layout
 * mlx_lm.convert writes (1: the zero-centred norms hold 1 + w, and a loader
 * hands the kernels stored - 1). Any other shape is refused. */
TESSL_API int32_t tessl_mlx_norm_convention_from_conv_shape(const char *tensor, const uint64_t *shape, uint32_t ndim,
                                                  uint64_t conv_dim, uint64_t kernel, uint32_t *convention, char *err,
                                                  size_t err_len);

/* `classify_outside` (src/qwen35_q4.rs:338-373): the tensors outside the tower's
 * prefix that no read touched: classes[i] = 0 for `mtp.*`, 1 for the vision
 * tower (skipped on purpose, by name); anything else is refused with its count
 * and the first eight names. */
TESSL_API int32_t tessl_mlx_classify_outside(const char *const *names, uint64_t n, uint8_t *classes, char *err,
                                   size_t err_len);

/* `check_part` (src/qwen35_q4.rs:384-449): the three tensors of one quantized
 * [rows, cols] matrix - `X.weight` U32 [rows, cols/8], `X.scales` and `X.biases`
 * BF16 [rows, cols/64] - checked by their headers alone, before any allocation. */
TESSL_API int32_t tessl_mlx_q4_check_part(const TesslCheckpoint *ck, const char *weight_name, uint64_t rows, uint64_t cols,
                                char *err, size_t err_len);

/* `Loader::mlx_q4_named` (src/loader.rs:256-318) into HOST memory: the parts'
 * rows one after the other ([q; k; v], [gate; up]), packed words unchanged,
 * scales and biases interleaved into bf16 (scale, bias) pairs; an infinite or
 * NaN scale or bias is refused by tensor, element, row and group. Every part is
 * checked before the first byte is written. */
TESSL_API int32_t tessl_mlx_q4_read_bank(const TesslCheckpoint *ck, const char *const *weight_names, const uint64_t *rows,
                               uint32_t nparts, uint64_t cols, void *packed, uint64_t packed_bytes, void *scales_biases,
                               uint64_t scales_biases_bytes, char *err, size_t err_len);

/* The same, into a bank whose device buffers the caller allocated (the
 * reference allocates inside; here allocation stays with the host framework).
 * Synchronises the runtime's stream before returning. */
TESSL_API int32_t tessl_mlx_q4_load_bank(TesslRuntime *rt, const TesslCheckpoint *ck, const char *const *weight_names,
                               const uint64_t *rows, uint32_t nparts, uint64_t cols, TesslQ4MlxBank bank, char *err,
                               size_t err_len);

/* ----------------------------------------------------- offline repack --- */

/* The B200 staged layout of one MLX Q4 bank [rows, cols], cols in {1024, 2048,
 * 4096}, group_size in {32, 64, 128}: NO COUNTERPART IN THE REFERENCE (its own
 * repack, Interleaved4, serves Apple GPUs: kernels/q4_mlx_dot.h:28-31). The bank
 * becomes ceil(rows / 8) units of 8 rows, each unit the exact bytes the GEMV kernel
 * keeps in shared memory: four pairs of adjacent packed rows (row 2i, row 2i + 1,
 * then 32 zero bytes), then the eight rows' (scale, bias) pairs; rows past the end
 * are zeros. A stage of the kernel is then two bulk copies instead of nine or
 * ten. The nibbles and pairs themselves are unchanged, and so is every result:
 * an entry given a staged bank returns the bits it returns for the row-major bank.
 * tessl_q4_mlx_staged_bytes gives the size (0 for a shape outside the domain);
 * tessl_q4_mlx_repack_staged writes the staged image of `bank` into `out`.
 * A staged bank is passed as TesslQ4MlxBank{packed = the image, scales_biases =
 * {NULL, 0}} with layout TESSL_Q4_B200_STAGED to tessl_gemv_q4_mlx_simd[_bf16],
 * tessl_gemv_q4_mlx_gate_up_gelu and tessl_gemv_q4_mlx_gate_up_silu_layout; the
 * other entries refuse it by name. */
TESSL_API uint64_t tessl_q4_mlx_staged_bytes(uint32_t rows, uint32_t cols, uint32_t group_size);
TESSL_API int32_t tessl_q4_mlx_repack_staged(TesslRuntime *rt, TesslQ4MlxBank bank, TesslQuantShape shape, TesslBuf out,
                                   char *err, size_t err_len);
/* tessl_gemv_q4_mlx_gate_up_silu with a layout argument (the reference's SiLU
 * entry is row-major only, src/nn.rs:4165-4194). */
TESSL_API int32_t tessl_gemv_q4_mlx_gate_up_silu_layout(TesslRuntime *rt, TesslQ4MlxBank gate, TesslQ4MlxBank up,
                                              TesslBuf x_bf16, TesslBuf mid, TesslQuantShape shape, uint32_t layout,
                                              uint32_t mid_as_bf16, char *err, size_t err_len);

/* ------------------------------------------------------- parity helpers --- */

/* Debug kernels for the bit-exact parity gates: the bank's nibbles as one
 * byte each [rows, cols], and its dense f32 image w = scale * q + bias
 * (separate multiply and add) [rows, cols]. */
TESSL_API int32_t tessl_q4_mlx_unpack(TesslRuntime *rt, TesslQ4MlxBank bank, TesslQuantShape shape, TesslBuf out_u8, char *err,
                            size_t err_len);
TESSL_API int32_t tessl_q4_mlx_dequant(TesslRuntime *rt, TesslQ4MlxBank bank, TesslQuantShape shape, TesslBuf out_f32,
                             char *err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* TESSL_B200_H */
