// `Q4Weight::{matmul, gate_up_silu}` of the reference (src/qwen35_q4.rs:518-611
// in the reference project): the policy that routes one group-64 MLX Q4 bank to
// the GEMV, the small-batch kernel or the tensor-core GEMM by the number of
// activation rows. Host code only.
#include "runtime.h"

namespace tessl {
namespace q4_weight {

namespace {
constexpr uint32_t kMlxQ4Group = 64;  // MLX_Q4_GROUP: the one group size Qwen3.5 checkpoints use
}

Result matmul(TesslRuntime *rt, const TesslQ4MlxBank &bank, uint32_t rows, uint32_t cols, const TesslBuf &x_bf16,
              uint32_t m, const TesslBuf &y, const TesslBuf *resid)
{
    const char *what = "Q4Weight::matmul";
    if (cols % kMlxQ4Group != 0)
        return fmt("Q4Weight: %u x %u does not fit a group-%u bank", rows, cols, kMlxQ4Group);
    // The reference checks tensor shapes; here the capacities stand in for them.
    if (x_bf16.nbytes / 2 < elems(m, cols) || y.nbytes / 4 < elems(m, rows)) {
        return fmt("%s: x [%u, %u] and y [%u, %u] do not fit a [%u, %u] weight", what, m, cols, m, rows, rows, cols);
    }
    const TesslQuantShape shape{rows, cols, kMlxQ4Group};
    if (m == 0) return ok();
    if (m == 1) return nn::gemv_q4_mlx_simd(rt, bank, x_bf16, y, shape, TESSL_Q4_ROW_MAJOR, resid, nn::OUT_F32);
    if (m <= TESSL_GEMM_Q4_MLX_MAX_M)
        return nn::gemm_q4_mlx(rt, bank, x_bf16, y, shape, m, TESSL_Q4_ROW_MAJOR, resid, nn::OUT_F32);
    if (resid)
        return fmt("%s: %u rows run on the TensorOps GEMM, which has no fused residual add", what, m);
    return nn::gemm_q4_mlx_tensorops(rt, bank, x_bf16, y, shape, m, nn::OUT_F32);
}

Result gate_up_silu(TesslRuntime *rt, const TesslQ4MlxBank &gate, const TesslQ4MlxBank &up, uint32_t rows,
                    uint32_t cols, const TesslBuf &x_bf16, const TesslBuf &mid, bool mid_as_bf16)
{
    const char *what = "Q4Weight::gate_up_silu";
    if (cols % kMlxQ4Group != 0)
        return fmt("Q4Weight: %u x %u does not fit a group-%u bank", rows, cols, kMlxQ4Group);
    if (x_bf16.nbytes / 2 < cols || mid.nbytes / (mid_as_bf16 ? 2 : 4) < rows) {
        return fmt("%s: x [1, %u] and mid [1, %u] do not fit a [%u, %u] weight at one row", what, cols, rows, rows,
                   cols);
    }
    const TesslQuantShape shape{rows, cols, kMlxQ4Group};
    return nn::gemv_q4_mlx_gate_up(rt, "gemv_q4_mlx_simd_gate_up_silu", "gemv_q4_mlx_gate_up_silu", true, gate, up,
                                   x_bf16, mid, shape, TESSL_Q4_ROW_MAJOR, mid_as_bf16);
}

}  // namespace q4_weight
}  // namespace tessl
