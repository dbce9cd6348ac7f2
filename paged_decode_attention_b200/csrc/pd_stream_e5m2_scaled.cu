// Streaming decode kernel instantiations for fp8_e5m2 pages with per-(token, head) scales.
#include "pd_stream_launch.cuh"

namespace pd {

cudaError_t stream_launch_e5m2_scaled(int head_dim, int hb, const StreamParams& sp, const CUtensorMap& mk,
                                 const CUtensorMap& mv, int grid, uint32_t smem, cudaStream_t st) {
  return launch_dtype<PD_KV_E5M2, true>(head_dim, hb, sp, mk, mv, grid, smem, st);
}

}  // namespace pd
