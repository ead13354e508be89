// All-gather of small per-GPU output slices over NVLink peer memory.
//
// The column-sharded GEMVs leave a few KB to a few hundred KB per GPU; a
// library all-gather of that size is pure latency (measured ~14 us per call
// inside a CUDA graph on two B200s, more than the sharded GEMV it follows).
// Here every rank owns one gather buffer in peer-mapped memory, the GEMV writes
// its slice straight into the buffer's own part, and one small kernel per rank
//   1. tells every peer it has arrived (so the peer's previous readers of the
//      buffer have finished: they precede the peer's gather in stream order) and
//      waits for every peer's arrival,
//   2. stores its slice into every peer's buffer (plain 16-byte peer stores),
//   3. tells every peer its slice is complete and waits for every peer's
//      completion. A system-scope fence (or an acquire or release at that scope)
//      costs ~1.8 us here, so there is exactly one per launch: every block
//      orders its stores before its ticket at device scope, and the block that
//      draws the last ticket fences once at system scope (cumulative over the
//      tickets it observed) before a relaxed store of the flag. Polls are
//      relaxed too: what they announce is read by later kernels of the stream.
// Flags are monotonically increasing call numbers kept in peer-mapped memory
// (`flags` of rank r: [0, 8) arrivals by source rank, [8, 16) completions by
// source rank, [16] this rank's own call counter, [17] a ticket counter of the
// call's thread blocks), so the same launch can be replayed from a CUDA graph.
// Larger slices are copied by several thread blocks; the last one to finish its
// part (by ticket) does the completion handshake. Every wait is bounded (~0.5 s unless the runtime's
// peer-wait limit says otherwise); on expiry the runtime's status word is set and the kernel returns. There is no counterpart
// in the reference (a single-device library).
#include <algorithm>

#include "runtime.h"

namespace tessl {
namespace {

struct PeerGatherParams {
    uint8_t *buf[8];     // gather buffer of every rank (this rank's own included), world * bytes_per_rank bytes each
    uint32_t *flags[8];  // flag words of every rank
    uint32_t rank, world;
    uint64_t bytes_per_rank;  // multiple of 16
    long long wait_clocks;    // bound of every wait for a peer
    uint32_t *status;
};

__device__ __forceinline__ void st_relaxed_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

/// Thread t < world (t != rank) waits until flag word `base + t` of this rank has reached `seq`.
__device__ __forceinline__ bool wait_peers(const PeerGatherParams &p, uint32_t base, uint32_t seq, uint32_t code)
{
    bool ok_ = true;
    if (threadIdx.x < p.world && threadIdx.x != p.rank) {
        const uint32_t *f = p.flags[p.rank] + base + threadIdx.x;
        const long long t0 = clock64();
        while ((int32_t)(ld_relaxed_sys(f) - seq) < 0) {
            if (clock64() - t0 > p.wait_clocks) {
                *(volatile uint32_t *)p.status = (0x50u << 24) | (code << 16) | threadIdx.x;
                ok_ = false;
                break;
            }
            __nanosleep(64);
        }
    }
    return __syncthreads_and(ok_) != 0;
}

__global__ void __launch_bounds__(1024, 1) peer_gather_kernel(const PeerGatherParams p)
{
    // Launched with programmatic stream serialization: the next kernel of the stream (a GEMV whose
    // weight stream does not depend on this exchange) may start its prologue now. This kernel may
    // itself have started before its predecessors finished, so it does nothing before the wait:
    // both the slice and "this rank's earlier readers of the buffer are done" need them complete.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t *mine = p.flags[p.rank];
    // This call's number, the same on every rank. [16] is only advanced by the call's last block, after every
    // block has read it here (a block takes its ticket after this read).
    const uint32_t seq = *(volatile uint32_t *)(mine + 16) + 1;
    // 1. arrival: block 0 tells the peers, every block waits for theirs
    if (blockIdx.x == 0 && threadIdx.x < p.world && threadIdx.x != p.rank)
        st_relaxed_sys(p.flags[threadIdx.x] + p.rank, seq);  // announces no data of this kernel
    if (!wait_peers(p, 0, seq, 1)) return;
    // 2. this rank's slice into every peer's buffer, the blocks sharing the 16-byte pieces
    const uint64_t n16 = p.bytes_per_rank / 16;
    const uint4 *src = reinterpret_cast<const uint4 *>(p.buf[p.rank] + (size_t)p.rank * p.bytes_per_rank);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        for (uint32_t r = 0; r < p.world; ++r)
            if (r != p.rank) reinterpret_cast<uint4 *>(p.buf[r] + (size_t)p.rank * p.bytes_per_rank)[i] = v;
    }
    __threadfence();
    __syncthreads();
    // 3. completion, by the last block to get here
    __shared__ uint32_t ticket;
    if (threadIdx.x == 0) ticket = atomicAdd(mine + 17, 1u);
    __syncthreads();
    if (ticket != gridDim.x - 1) return;
    // every block's stores precede its ticket at device scope, all tickets were observed here: this one fence
    // puts them all before the flag at system scope
    if (threadIdx.x < 32) __threadfence_system();
    __syncthreads();
    if (threadIdx.x < p.world && threadIdx.x != p.rank) st_relaxed_sys(p.flags[threadIdx.x] + 8 + p.rank, seq);
    if (!wait_peers(p, 8, seq, 2)) return;
    if (threadIdx.x == 0) mine[17] = 0, mine[16] = seq;
}

/// The wait that a deferred exchange left to its reader, as a launch of its own (for readers that are not the
/// tensor-core GEMV, which does it itself): every peer's completion flag has reached this rank's call counter.
__global__ void peer_wait_kernel(const uint32_t *mine, uint32_t rank, uint32_t world, long long wait_clocks, uint32_t *status)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t seq = *(volatile const uint32_t *)(mine + 16);
    if (threadIdx.x < world && threadIdx.x != rank) {
        const long long t0 = clock64();
        while ((int32_t)(ld_relaxed_sys(mine + 8 + threadIdx.x) - seq) < 0) {
            if (clock64() - t0 > wait_clocks) {
                *(volatile uint32_t *)status = (0x50u << 24) | (5u << 16) | threadIdx.x;
                break;
            }
            __nanosleep(64);
        }
    }
}

}  // namespace

namespace nn {

Result peer_wait(TesslRuntime *rt, const TesslPeerGather &g)
{
    TESSL_TRY(peer_gather_validate(g, "peer_wait"));
    if (g.world == 1) return ok();
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(1), lc.blockDim = dim3(32), lc.dynamicSmemBytes = 0;
    lc.stream = rt->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr, lc.numAttrs = 1;
    const long long clocks = rt->peer_wait_clocks ? (long long)rt->peer_wait_clocks : kPeerWaitClocks;
    const cudaError_t e = cudaLaunchKernelEx(&lc, peer_wait_kernel, (const uint32_t *)g.flags[g.rank], g.rank, g.world, clocks,
                                             rt->status_dev);
    rt->dispatch_count += 1;
    return cuda_check(rt, e, "peer_wait launch");
}

Result peer_gather(TesslRuntime *rt, const TesslPeerGather &g)
{
    TESSL_TRY(peer_gather_validate(g, "peer_gather"));
    if (g.world == 1 || g.bytes_per_rank == 0) return ok();
    PeerGatherParams p{};
    for (uint32_t r = 0; r < g.world; ++r) p.buf[r] = static_cast<uint8_t *>(g.buffers[r]), p.flags[r] = g.flags[r];
    p.rank = g.rank, p.world = g.world, p.bytes_per_rank = g.bytes_per_rank;
    p.wait_clocks = rt->peer_wait_clocks ? (long long)rt->peer_wait_clocks : kPeerWaitClocks;
    p.status = rt->status_dev;
    cudaLaunchConfig_t lc{};
    // one block per 32 KiB of slice, at most 16: a few KB go fastest from one block, the LM head's
    // hundreds of KB need several to fill the link
    const uint32_t blocks = (uint32_t)std::min<uint64_t>(16, std::max<uint64_t>(1, g.bytes_per_rank / 32768));
    lc.gridDim = dim3(blocks), lc.blockDim = dim3(1024), lc.dynamicSmemBytes = 0;
    lc.stream = rt->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr, lc.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&lc, peer_gather_kernel, p);
    rt->dispatch_count += 1;
    return cuda_check(rt, e, "peer_gather launch");
}

}  // namespace nn
}  // namespace tessl
