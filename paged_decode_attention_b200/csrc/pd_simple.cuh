// General decode kernel: one CTA per (kv head x query-head chunk, request, split).
//
// CUDA cores only, plain vector loads, any element strides, every head_dim in
// {32, 64, 128, 256}, every kv dtype, any group size.  It is the path for shapes and
// strides the streaming kernel does not serve and the A/B partner for it.  Each warp walks
// the tokens of the range with a stride of four; a lane owns head_dim / 32 contiguous
// elements of the row, so one warp-wide load covers a whole K (or V) row; the dot products
// of up to eight query heads of the group are reduced with warp shuffles and fed to a base-2
// online softmax (the reference's recurrence, pagedattn/triton_decode.py:159-166).  The four
// warps' states are merged through shared memory at the end.
#pragma once

#include "pd_common.cuh"

namespace pd {

constexpr int kSimpleWarps = 4;
constexpr int kSimpleThreads = kSimpleWarps * 32;

template <int D>
__host__ __device__ constexpr int simple_heads_per_cta() {
  return D <= 128 ? 8 : 4;
}

template <int KV, int D, bool IO_BF16, bool SCALED>
__global__ void __launch_bounds__(kSimpleThreads)
simple_decode_kernel(const Params p) {
  constexpr int EPL = D / 32;                  // elements per lane
  constexpr int GH = simple_heads_per_cta<D>();  // query heads per CTA
  const int chunks = (p.group + GH - 1) / GH;
  const int kvh = blockIdx.x / chunks;
  const int g0 = (blockIdx.x % chunks) * GH;   // first group member handled here
  const int gn = min(GH, p.group - g0);
  const int b = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int seq_len = clamp_len(p, b);
  int lo, hi;
  split_range(seq_len, split, p.num_splits, p.block_n, lo, hi);

  float q[GH][EPL];
#pragma unroll
  for (int g = 0; g < GH; ++g) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      q[g][e] = 0.f;
      if (g < gn)
        q[g][e] = io_to_float<IO_BF16>(p.q, (int64_t)b * p.q_sb +
                                                 (int64_t)(kvh * p.group + g0 + g) * p.q_sh +
                                                 lane * EPL + e);
    }
  }

  float m[GH], l[GH], acc[GH][EPL];
#pragma unroll
  for (int g = 0; g < GH; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }

  for (int t = lo + warp; t < hi; t += kSimpleWarps) {
    const int blk = lookup_block(p, b, t / p.page);
    if (blk < 0) continue;
    const int slot = t % p.page;
    const int64_t row = kv_row_offset(p, blk, slot, kvh) + lane * EPL;
    float kf[EPL], vf[EPL];
    load_elems<KV, EPL>(p.k, row, kf);
    load_elems<KV, EPL>(p.v, row, vf);
    if constexpr (SCALED) {
      const int64_t so = scale_offset(p, blk, slot, kvh);
      const float ks = __half2float(__ldg(p.k_scale + so));
      const float vs = __half2float(__ldg(p.v_scale + so));
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        kf[e] = apply_scale_fp16(kf[e], ks);
        vf[e] = apply_scale_fp16(vf[e], vs);
      }
    }
#pragma unroll
    for (int g = 0; g < GH; ++g) {
      if (g < gn) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) s = fmaf(q[g][e], kf[e], s);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s *= p.scale_log2;
        const float m_new = fmaxf(m[g], s);
        const float alpha = fast_exp2(m[g] - m_new);  // exp2(-inf) = 0 on the first token
        const float w = fast_exp2(s - m_new);
        l[g] = l[g] * alpha + w;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = fmaf(acc[g][e], alpha, w * vf[e]);
        m[g] = m_new;
      }
    }
  }

  // merge the warps' (m, l, acc) states
  __shared__ float sm_m[kSimpleWarps][GH];
  __shared__ float sm_l[kSimpleWarps][GH];
  __shared__ float sm_acc[kSimpleWarps][GH][D];
#pragma unroll
  for (int g = 0; g < GH; ++g) {
    if (lane == 0) {
      sm_m[warp][g] = m[g];
      sm_l[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_acc[warp][g][lane * EPL + e] = acc[g][e];
  }
  __syncthreads();

  for (int idx = threadIdx.x; idx < gn * D; idx += kSimpleThreads) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kSimpleWarps; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, oo = 0.f;
    if (mm > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kSimpleWarps; ++w) {
        const float f = fast_exp2(sm_m[w][g] - mm);
        ll += sm_l[w][g] * f;
        oo += sm_acc[w][g][d] * f;
      }
    }
    const float o = ll > 0.f ? oo / ll : 0.f;
    const float lse = ll > 0.f ? mm + log2f(ll) : -INFINITY;
    const int hq = kvh * p.group + g0 + g;
    if (p.num_splits > 1) {
      // scratch layout [split][request * Hq + head][D]
      const int64_t r = (int64_t)split * p.batch * p.hq + (int64_t)b * p.hq + hq;
      p.part_o[r * D + d] = o;
      if (d == 0) p.part_lse[r] = lse;
    } else {
      if (p.out) io_store<IO_BF16>(p.out, (int64_t)b * p.o_sb + (int64_t)hq * p.o_sh + d, o);
      if (p.res_o) {
        p.res_o[((int64_t)b * p.hq + hq) * D + d] = o;
        if (d == 0) p.res_lse[(int64_t)b * p.hq + hq] = lse;
      }
    }
  }
}

}  // namespace pd
