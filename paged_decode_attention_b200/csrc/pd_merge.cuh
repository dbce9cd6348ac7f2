// Log-sum-exp merge of partial attention results and the dense debug gather.
#pragma once

#include "pd_common.cuh"

namespace pd {

struct MergeParams {
  const float* part_o;
  const float* part_lse;
  int64_t o_sp, o_sr, l_sp, l_sr;
  int32_t parts, rows, d;
  void* out;        // row r is written at (r / rows_per_batch) * dst_sb + (r % rows_per_batch) * dst_sh
  int64_t dst_sb, dst_sh;
  int32_t rows_per_batch;
  float* res_o;
  float* res_lse;
};

// One CTA per row (request x query head).  Partials are normalised results with base-2
// log-sum-exps, so merged = sum_p 2^(lse_p - m) o_p / sum_p 2^(lse_p - m) with m = max lse
// (pagedattn/triton_decode.py:221-240).  Rows whose partials are all empty (-inf) become
// zero with lse -inf instead of the reference's 0/0.
template <bool IO_BF16>
__global__ void __launch_bounds__(128) merge_kernel(const MergeParams p) {
  const int row = blockIdx.x;
  const int64_t dst = (int64_t)(row / p.rows_per_batch) * p.dst_sb +
                      (int64_t)(row % p.rows_per_batch) * p.dst_sh;
  float m = -INFINITY;
  for (int i = 0; i < p.parts; ++i)
    m = fmaxf(m, __ldg(p.part_lse + (int64_t)i * p.l_sp + (int64_t)row * p.l_sr));
  float denom = 0.f;
  if (m > -INFINITY)
    for (int i = 0; i < p.parts; ++i)
      denom += exp2f(__ldg(p.part_lse + (int64_t)i * p.l_sp + (int64_t)row * p.l_sr) - m);
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int d = threadIdx.x; d < p.d; d += blockDim.x) {
    float acc = 0.f;
    if (denom > 0.f) {
      for (int i = 0; i < p.parts; ++i) {
        const float lse = __ldg(p.part_lse + (int64_t)i * p.l_sp + (int64_t)row * p.l_sr);
        if (lse > -INFINITY)
          acc += exp2f(lse - m) * __ldg(p.part_o + (int64_t)i * p.o_sp + (int64_t)row * p.o_sr + d);
      }
    }
    const float o = acc * inv;
    if (p.out) io_store<IO_BF16>(p.out, dst + d, o);
    if (p.res_o) p.res_o[(int64_t)row * p.d + d] = o;
  }
  if (threadIdx.x == 0 && p.res_lse) p.res_lse[row] = denom > 0.f ? m + log2f(denom) : -INFINITY;
}

// Dense [B][Hkv][s_max][D] fp16 copy of the dequantised pages, one warp per row; rows at or
// past a request's length are zero.  Shares lookup_block / kv_row_offset / apply_scale_fp16
// with the decode kernels.
template <int KV, int D, bool SCALED>
__global__ void __launch_bounds__(128)
gather_kernel(const Params p, __half* __restrict__ k_dense, __half* __restrict__ v_dense, int s_max) {
  constexpr int EPL = D / 32;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int64_t total = (int64_t)p.batch * p.hkv * s_max;
  if (row >= total) return;
  const int s = (int)(row % s_max);
  const int h = (int)((row / s_max) % p.hkv);
  const int b = (int)(row / ((int64_t)s_max * p.hkv));
  float kf[EPL], vf[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) kf[e] = vf[e] = 0.f;
  if (s < clamp_len(p, b)) {
    const int blk = lookup_block(p, b, s / p.page);
    if (blk >= 0) {
      const int slot = s % p.page;
      const int64_t src = kv_row_offset(p, blk, slot, h) + lane * EPL;
      load_elems<KV, EPL>(p.k, src, kf);
      load_elems<KV, EPL>(p.v, src, vf);
      if constexpr (SCALED) {
        const int64_t so = scale_offset(p, blk, slot, h);
        const float ks = __half2float(__ldg(p.k_scale + so));
        const float vs = __half2float(__ldg(p.v_scale + so));
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          kf[e] = apply_scale_fp16(kf[e], ks);
          vf[e] = apply_scale_fp16(vf[e], vs);
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    k_dense[row * D + lane * EPL + e] = __float2half_rn(kf[e]);
    v_dense[row * D + lane * EPL + e] = __float2half_rn(vf[e]);
  }
}

}  // namespace pd
