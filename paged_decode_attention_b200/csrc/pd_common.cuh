// Shared device-side definitions of the paged decode kernels: the launch parameter block,
// the page address function and the stored-element conversions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/paged_decode.h"

namespace pd {

constexpr float kLog2e = 1.4426950408889634f;

// Device view of PdDecodeArgs with derived values filled in by the host.
struct Params {
  const void* q;
  void* out;
  int64_t q_sb, q_sh, o_sb, o_sh;
  const void* k;
  const void* v;
  int64_t kv_sb, kv_st, kv_sh;  // element strides: block, token, head
  const __half* k_scale;
  const __half* v_scale;
  int64_t sc_sb, sc_st;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* seq_lens;
  int32_t batch, hq, hkv, d, page, num_blocks, max_blocks, group;
  float scale_log2;  // sm_scale * log2(e): softmax runs in base 2
  int32_t num_splits, block_n;
  float* part_o;    // split scratch
  float* part_lse;
  float* res_o;     // optional fp32 result + lse
  float* res_lse;
  uint32_t* status;
};

// Token range [lo, hi) of one split of a request: the reference's rule
// (pagedattn/triton_decode.py:78-82): chunks of ceil(ceil(len / block_n) / splits) tiles.
__host__ __device__ inline void split_range(int seq_len, int split, int num_splits, int block_n,
                                            int& lo, int& hi) {
  if (num_splits <= 1) {
    lo = 0;
    hi = seq_len;
    return;
  }
  const int tiles = (seq_len + block_n - 1) / block_n;
  const int chunk = ((tiles + num_splits - 1) / num_splits) * block_n;
  const long long l = (long long)split * chunk;
  lo = l > seq_len ? seq_len : (int)l;
  hi = lo + chunk < seq_len ? lo + chunk : seq_len;
}

// Element offset of the K (or V) row of (physical block, token slot, kv head).  64-bit: a
// pool of more than 2^31 elements must not wrap (the reference indexes in 32 bits).
__device__ __forceinline__ int64_t kv_row_offset(const Params& p, int block, int token, int head) {
  return (int64_t)block * p.kv_sb + (int64_t)token * p.kv_st + (int64_t)head * p.kv_sh;
}

__device__ __forceinline__ int64_t scale_offset(const Params& p, int block, int token, int head) {
  return (int64_t)block * p.sc_sb + (int64_t)token * p.sc_st + head;
}

// Physical block of logical page `page_idx` of request b, or -1 (and a status bit) when the
// table holds an id outside the pool.
__device__ __forceinline__ int lookup_block(const Params& p, int b, int page_idx) {
  const int blk = __ldg(p.block_table + (int64_t)b * p.bt_stride + page_idx);
  if ((unsigned)blk >= (unsigned)p.num_blocks) {
    if (p.status) atomicOr(p.status, PD_DEV_BAD_BLOCK);
    return -1;
  }
  return blk;
}

// Length of request b as every kernel uses it: negative lengths count as zero, and a length
// beyond what the block-table row can name (max_blocks * page tokens) is cut there with
// PD_DEV_BAD_BLOCK raised, so a stale or oversized length never indexes past the row.
__device__ __forceinline__ int clamp_len(const Params& p, int b) {
  int len = __ldg(p.seq_lens + b);
  const long long cap = (long long)p.max_blocks * p.page;
  if (len < 0) len = 0;
  if (len > cap) {
    if (p.status) atomicOr(p.status, PD_DEV_BAD_BLOCK);
    len = (int)cap;
  }
  return len;
}

// fp16 value of a stored element, exact for every kv dtype except bf16 (rounded to nearest).
template <int KV>
struct Stored;
template <>
struct Stored<PD_KV_F16> {
  using type = __half;
  static constexpr int bytes = 2;
  __device__ static __forceinline__ float to_float(uint32_t bits) {
    return __half2float(__ushort_as_half((unsigned short)bits));
  }
};
template <>
struct Stored<PD_KV_BF16> {
  using type = __nv_bfloat16;
  static constexpr int bytes = 2;
  __device__ static __forceinline__ float to_float(uint32_t bits) {
    // the reference converts bf16 pages to fp16 first (pagedattn/cache.py:55-56)
    return __half2float(__float2half_rn(__uint_as_float(bits << 16)));
  }
};
template <>
struct Stored<PD_KV_E5M2> {
  using type = uint8_t;
  static constexpr int bytes = 1;
  __device__ static __forceinline__ float to_float(uint32_t bits) {
    // e5m2 is the high byte of an fp16 (pagedattn/cache.py:27-28)
    return __half2float(__ushort_as_half((unsigned short)(bits << 8)));
  }
};
template <>
struct Stored<PD_KV_I8> {
  using type = int8_t;
  static constexpr int bytes = 1;
  __device__ static __forceinline__ float to_float(uint32_t bits) { return (float)(int8_t)bits; }
};

// Loads N stored elements (N * bytes in {1,2,4,8,16}, naturally aligned) and widens them.
template <int KV, int N>
__device__ __forceinline__ void load_elems(const void* base, int64_t elem_off, float (&dst)[N]) {
  constexpr int kBytes = N * Stored<KV>::bytes;
  const char* ptr = (const char*)base + elem_off * Stored<KV>::bytes;
  uint32_t w[(kBytes + 3) / 4];
  if constexpr (kBytes == 16) {
    const uint4 t = __ldg((const uint4*)ptr);
    w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
  } else if constexpr (kBytes == 8) {
    const uint2 t = __ldg((const uint2*)ptr);
    w[0] = t.x; w[1] = t.y;
  } else if constexpr (kBytes == 4) {
    w[0] = __ldg((const uint32_t*)ptr);
  } else if constexpr (kBytes == 2) {
    w[0] = __ldg((const unsigned short*)ptr);
  } else {
    w[0] = __ldg((const unsigned char*)ptr);
  }
#pragma unroll
  for (int i = 0; i < N; ++i) {
    if constexpr (Stored<KV>::bytes == 2)
      dst[i] = Stored<KV>::to_float((w[i / 2] >> (16 * (i % 2))) & 0xffffu);
    else
      dst[i] = Stored<KV>::to_float((w[i / 4] >> (8 * (i % 4))) & 0xffu);
  }
}

// The reference's dequantisation: fp16(stored) * fp16 scale, rounded to fp16
// (pagedattn/cache.py:59-61).
__device__ __forceinline__ float apply_scale_fp16(float x, float s) {
  return __half2float(__float2half_rn(x * s));
}

template <bool BF16>
__device__ __forceinline__ float io_to_float(const void* base, int64_t idx) {
  if constexpr (BF16) return __bfloat162float(((const __nv_bfloat16*)base)[idx]);
  else return __half2float(((const __half*)base)[idx]);
}

template <bool BF16>
__device__ __forceinline__ void io_store(void* base, int64_t idx, float x) {
  if constexpr (BF16) ((__nv_bfloat16*)base)[idx] = __float2bfloat16_rn(x);
  else ((__half*)base)[idx] = __float2half_rn(x);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace pd
