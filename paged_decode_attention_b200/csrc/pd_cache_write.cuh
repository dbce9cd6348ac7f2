// Writes one step's keys and values into the paged cache, quantising on the way.
//
// The step before the decode path: the reference's backend calls vLLM's
// reshape_and_cache_flash (integration/vllm_backend.py:117-122) and its fixtures quantise with
// quantize_kv (pagedattn/cache.py:33-48).  This kernel does both at once for the NHD layout the
// decode kernels read: row (token, kv head) of `key`/`value` goes to slot
// slot_mapping[token] = block * block_size + offset of k_cache/v_cache; a negative slot (padding)
// is skipped; a slot outside the pool sets PD_DEV_BAD_BLOCK and is skipped.
//
// Quantisation is bit-exact with the reference's rules:
//   int8:      scale = fp16(max(amax, 1e-6) / 127),  q = clamp(rint(x / scale), -127, 127)
//              (fp32 division, round half to even; 0/0 from an all-zero row stores 0)
//   fp8_e5m2:  round to nearest even on the fp16 bits, overflow to infinity, no scale
//   16-bit:    a cast
// One warp per (token, kv head); a lane owns head_dim / 32 contiguous elements.
#pragma once

#include "pd_common.cuh"

namespace pd {

struct CacheWriteParams {
  const void* key;
  const void* value;
  int64_t in_st, in_sh;  // element strides of key/value: token, head
  void* k_cache;
  void* v_cache;
  int64_t kv_sb, kv_st, kv_sh;
  __half* k_scale;
  __half* v_scale;
  int64_t sc_sb, sc_st;
  const int64_t* slot_mapping;
  int32_t num_tokens, hkv, d, page, num_blocks;
  uint32_t* status;
};

// fp16 bits -> e5m2 bits, round to nearest even (what a cast to float8_e5m2 does).
__device__ __forceinline__ uint8_t half_bits_to_e5m2(uint32_t h) {
  if ((h & 0x7fffu) > 0x7c00u) return (uint8_t)((h >> 8) | 0x02u);  // NaN stays NaN
  return (uint8_t)((h + 0x7fu + ((h >> 8) & 1u)) >> 8);
}

template <int KV, int D, bool IO_BF16>
__global__ void __launch_bounds__(128) cache_write_kernel(const CacheWriteParams p) {
  constexpr int EPL = D / 32;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (int64_t)p.num_tokens * p.hkv) return;
  const int token = (int)(row / p.hkv), head = (int)(row % p.hkv);
  const int64_t slot = p.slot_mapping[token];
  if (slot < 0) return;
  if (slot >= (int64_t)p.num_blocks * p.page) {
    if (p.status && lane == 0) atomicOr(p.status, PD_DEV_BAD_BLOCK);
    return;
  }
  const int block = (int)(slot / p.page), off = (int)(slot % p.page);
  const int64_t src = (int64_t)token * p.in_st + (int64_t)head * p.in_sh + lane * EPL;
  const int64_t dst = (int64_t)block * p.kv_sb + (int64_t)off * p.kv_st + (int64_t)head * p.kv_sh + lane * EPL;

#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const void* in = which ? p.value : p.key;
    void* out = which ? p.v_cache : p.k_cache;
    float x[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) x[e] = io_to_float<IO_BF16>(in, src + e);
    if constexpr (KV == PD_KV_F16) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) ((__half*)out)[dst + e] = __float2half_rn(x[e]);
    } else if constexpr (KV == PD_KV_BF16) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) ((__nv_bfloat16*)out)[dst + e] = __float2bfloat16_rn(x[e]);
    } else if constexpr (KV == PD_KV_E5M2) {
#pragma unroll
      for (int e = 0; e < EPL; ++e)
        ((uint8_t*)out)[dst + e] = half_bits_to_e5m2(__half_as_ushort(__float2half_rn(x[e])));
      // the reference's fp8 cast has no scale; a cache that carries scales anyway gets 1
      if (lane == 0 && p.k_scale) {
        __half* sc = which ? p.v_scale : p.k_scale;
        sc[(int64_t)block * p.sc_sb + (int64_t)off * p.sc_st + head] = __float2half_rn(1.f);
      }
    } else {
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(x[e]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const __half scale_h = __float2half_rn(__fdiv_rn(fmaxf(amax, 1e-6f), 127.f));
      const float scale = __half2float(scale_h);
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float q = rintf(__fdiv_rn(x[e], scale));
        // 0/0 (an all-zero row whose scale underflowed) stores 0, as the reference's cast does
        ((int8_t*)out)[dst + e] = (q != q) ? (int8_t)0 : (int8_t)fminf(fmaxf(q, -127.f), 127.f);
      }
      if (lane == 0) {
        __half* sc = which ? p.v_scale : p.k_scale;
        sc[(int64_t)block * p.sc_sb + (int64_t)off * p.sc_st + head] = scale_h;
      }
    }
  }
}

}  // namespace pd
