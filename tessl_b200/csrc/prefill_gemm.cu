// placeholder replaced by the tcgen05 kernel
#include "runtime.h"
namespace tessl { namespace nn {
uint32_t gemm_q4_mlx_tensorops_max_k(uint32_t m, uint32_t n, uint32_t group_size)
{
    const uint64_t widest = std::max<uint64_t>(std::max(m, n), 1);
    const uint64_t k = std::min<uint64_t>(0x7fffffffull / widest, 0xffffffffull);
    const uint64_t g = std::max<uint32_t>(group_size, 1);
    return (uint32_t)(k / g * g);
}
Result gemm_q4_mlx_tensorops(TesslRuntime *, const TesslQ4MlxBank &, const TesslBuf &, const TesslBuf &,
                             const TesslQuantShape &, uint32_t, OutKind)
{
    return "gemm_q4_mlx_tensorops: not built yet";
}
}}
