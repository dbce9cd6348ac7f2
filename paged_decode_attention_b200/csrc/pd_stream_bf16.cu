// Streaming decode kernel instantiations for bf16 pages.
#include "pd_stream_launch.cuh"

namespace pd {

cudaError_t stream_launch_bf16(int head_dim, int hb, const StreamParams& sp, const CUtensorMap& mk,
                                 const CUtensorMap& mv, int grid, uint32_t smem, cudaStream_t st) {
  return launch_dtype<PD_KV_BF16, false>(head_dim, hb, sp, mk, mv, grid, smem, st);
}

}  // namespace pd
