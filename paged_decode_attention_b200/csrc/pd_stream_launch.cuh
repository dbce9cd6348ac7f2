// Kernel dispatch of the streaming decode: from the run-time shape (head_dim, heads per block,
// group size) to the template instantiation that serves it.  Included by one translation unit
// per page element type (pd_stream_<type>.cu), so the instantiations compile in parallel.
#pragma once

#include "pd_stream_kernel.cuh"

namespace pd {

template <int KV, int D, int HB, bool SCALED, int NG, int WPC>
static inline cudaError_t launch_wpc(const StreamParams& sp, const CUtensorMap& mk, const CUtensorMap& mv,
                              int grid, uint32_t smem, cudaStream_t st) {
  auto* kern = stream_decode_kernel<KV, D, HB, SCALED, NG, WPC>;
  static bool configured[64] = {};  // per device: the opt-in shared-memory limit has been raised
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return cudaErrorInvalidDevice;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  kern<<<grid, WPC * (HB + 1) * 32, smem, st>>>(sp, mk, mv);
  return cudaGetLastError();
}

template <int KV, int D, int HB, bool SCALED, int NG>
static inline cudaError_t launch_ng(const StreamParams& sp, const CUtensorMap& mk, const CUtensorMap& mv,
                             int grid, uint32_t smem, cudaStream_t st) {
  if constexpr (D == 256) {
    static_assert(HB <= 4, "head_dim 256 runs at most four heads per block");
    return launch_wpc<KV, D, HB, SCALED, NG, 4 / HB>(sp, mk, mv, grid, smem, st);
  } else {
    return launch_wpc<KV, D, HB, SCALED, NG, base_workers_per_cta(HB)>(sp, mk, mv, grid, smem, st);
  }
}

// groups of up to 8 query heads fit one 8-wide n-tile, up to 16 need two
template <int KV, int D, int HB, bool SCALED>
static inline cudaError_t launch_one(const StreamParams& sp, const CUtensorMap& mk, const CUtensorMap& mv,
                              int grid, uint32_t smem, cudaStream_t st) {
  return sp.p.group <= 8 ? launch_ng<KV, D, HB, SCALED, 1>(sp, mk, mv, grid, smem, st)
                         : launch_ng<KV, D, HB, SCALED, 2>(sp, mk, mv, grid, smem, st);
}

template <int KV, int D, bool SCALED>
static inline cudaError_t launch_hb(int hb, const StreamParams& sp, const CUtensorMap& mk, const CUtensorMap& mv,
                             int grid, uint32_t smem, cudaStream_t st) {
  switch (hb) {
    case 8:
      if constexpr (D != 256) return launch_one<KV, D, 8, SCALED>(sp, mk, mv, grid, smem, st);
      else return cudaErrorInvalidValue;
    case 4: return launch_one<KV, D, 4, SCALED>(sp, mk, mv, grid, smem, st);
    case 2: return launch_one<KV, D, 2, SCALED>(sp, mk, mv, grid, smem, st);
    default: return launch_one<KV, D, 1, SCALED>(sp, mk, mv, grid, smem, st);
  }
}

// Every head_dim the page type KV is served at.
template <int KV, bool SCALED>
static inline cudaError_t launch_dtype(int head_dim, int hb, const StreamParams& sp, const CUtensorMap& mk,
                                       const CUtensorMap& mv, int grid, uint32_t smem, cudaStream_t st) {
  switch (head_dim) {
    case 128: return launch_hb<KV, 128, SCALED>(hb, sp, mk, mv, grid, smem, st);
    case 256: return launch_hb<KV, 256, SCALED>(hb, sp, mk, mv, grid, smem, st);
    case 64: return launch_hb<KV, 64, SCALED>(hb, sp, mk, mv, grid, smem, st);
    case 32:
      if constexpr (is_16bit(KV)) return launch_hb<KV, 32, SCALED>(hb, sp, mk, mv, grid, smem, st);
      else return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace pd
