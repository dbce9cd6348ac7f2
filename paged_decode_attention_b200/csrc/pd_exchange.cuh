// Cross-GPU exchange of decode partials without a collective library: every rank stores its
// partial straight into every peer's exchange buffer over NVLink (plain peer stores, no
// multicast, no loads from peer memory), raises a flag there, and each rank merges what has
// landed in its own memory.  Used by the KV-range-sharded long-context path in place of
// all-gather + merge; the arithmetic is the log-sum-exp merge of
// pagedattn/triton_decode.py:221-240 over ranks instead of splits.
//
// Exchange buffer of one rank (identical layout on every rank, `n` = floats of one partial:
// rows * D normalised fp32 results followed by rows base-2 log-sum-exps):
//   [0]   uint32 step          steps this rank has merged
//   [1]   uint32 done_ticket   CTAs of the running merge that have finished
//   [16 + parity * kMaxRanks + r]  uint32 flag: step + 1 once rank r's partial of that step is here
//   byte 256 + (parity * world + r) * n * 4:  rank r's partial
// Two parities because a peer may run one step ahead of this rank, never two: its next push
// needs its own merge of this step, which needs this rank's flag of this step.
//
// Every wait is bounded (one second): on expiry the kernel sets PD_DEV_TIMEOUT in the status
// word, skips the merge and returns.
#pragma once

#include "pd_common.cuh"

namespace pd {

constexpr int kMaxRanks = 16;
constexpr int kExchangeHeaderBytes = 256;
constexpr unsigned long long kExchangeWaitNs = 1000000000ull;

struct PeerPointers {
  unsigned char* buf[kMaxRanks];
};

__host__ __device__ inline uint64_t exchange_bytes(int world, int64_t n) {
  return kExchangeHeaderBytes + (uint64_t)2 * world * n * 4;
}

__device__ __forceinline__ uint32_t* exchange_flag(unsigned char* buf, int parity, int r) {
  return reinterpret_cast<uint32_t*>(buf) + 16 + parity * kMaxRanks + r;
}
__device__ __forceinline__ float* exchange_part(unsigned char* buf, int world, int64_t n, int parity, int r) {
  return reinterpret_cast<float*>(buf + kExchangeHeaderBytes) + ((int64_t)parity * world + r) * n;
}

// One CTA per destination rank: copy this rank's partial into the destination's slot for this
// rank, make it visible system-wide, then publish the flag.
__global__ void __launch_bounds__(256)
exchange_push_kernel(const float* __restrict__ local, PeerPointers peers, int world, int rank, int64_t n) {
  const int dst = blockIdx.x;
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(peers.buf[rank]);
  const int parity = step & 1u;
  float* out = exchange_part(peers.buf[dst], world, n, parity, rank);
  const int64_t n4 = n / 4;
  const float4* src4 = reinterpret_cast<const float4*>(local);
  float4* out4 = reinterpret_cast<float4*>(out);
  for (int64_t i = threadIdx.x; i < n4; i += blockDim.x) out4[i] = src4[i];
  for (int64_t i = 4 * n4 + threadIdx.x; i < n; i += blockDim.x) out[i] = local[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* flag = exchange_flag(peers.buf[dst], parity, rank);
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(step + 1u) : "memory");
  }
}

struct ExchangeMergeParams {
  unsigned char* buf;  // this rank's exchange buffer
  int32_t world, rows, d, rows_per_batch;
  void* out;
  int64_t dst_sb, dst_sh;
  float* res_o;
  float* res_lse;
  uint32_t* status;
};

// One CTA per row (request x query head): wait (bounded) until every rank's partial of this
// step has landed here, merge them, and let the last CTA advance the step.
template <bool IO_BF16>
__global__ void __launch_bounds__(128) exchange_merge_kernel(const ExchangeMergeParams p) {
  __shared__ int ok;
  uint32_t* header = reinterpret_cast<uint32_t*>(p.buf);
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(header);
  const int parity = step & 1u;
  const int64_t n = (int64_t)p.rows * (p.d + 1);
  if (threadIdx.x == 0) {
    int good = 1;
    unsigned long long t0 = 0;
    for (int r = 0; r < p.world && good; ++r) {
      const uint32_t* flag = exchange_flag(p.buf, parity, r);
      unsigned spins = 0;
      for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v == step + 1u) break;
        if ((++spins & 63u) == 0) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (t0 == 0) t0 = now;
          if (now - t0 > kExchangeWaitNs) {
            if (p.status) atomicOr(p.status, PD_DEV_TIMEOUT);
            good = 0;
            break;
          }
        }
      }
    }
    ok = good;
  }
  __syncthreads();
  const int row = blockIdx.x;
  if (ok) {
    float m = -INFINITY;
    for (int r = 0; r < p.world; ++r)
      m = fmaxf(m, __ldcg(exchange_part(p.buf, p.world, n, parity, r) + (int64_t)p.rows * p.d + row));
    float denom = 0.f;
    if (m > -INFINITY)
      for (int r = 0; r < p.world; ++r) {
        const float lse = __ldcg(exchange_part(p.buf, p.world, n, parity, r) + (int64_t)p.rows * p.d + row);
        if (lse > -INFINITY) denom += exp2f(lse - m);
      }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    const int64_t dst = (int64_t)(row / p.rows_per_batch) * p.dst_sb + (int64_t)(row % p.rows_per_batch) * p.dst_sh;
    for (int d = threadIdx.x; d < p.d; d += blockDim.x) {
      float acc = 0.f;
      if (denom > 0.f)
        for (int r = 0; r < p.world; ++r) {
          const float* part = exchange_part(p.buf, p.world, n, parity, r);
          const float lse = __ldcg(part + (int64_t)p.rows * p.d + row);
          if (lse > -INFINITY) acc += exp2f(lse - m) * __ldcg(part + (int64_t)row * p.d + d);
        }
      const float o = acc * inv;
      if (p.out) io_store<IO_BF16>(p.out, dst + d, o);
      if (p.res_o) p.res_o[(int64_t)row * p.d + d] = o;
    }
    if (threadIdx.x == 0 && p.res_lse) p.res_lse[row] = denom > 0.f ? m + log2f(denom) : -INFINITY;
  }
  // the last CTA to finish closes the step; every CTA read `step` before taking its ticket
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(header + 1, 1u) == gridDim.x - 1) {
      header[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(header) = step + 1u;
    }
  }
}

}  // namespace pd
