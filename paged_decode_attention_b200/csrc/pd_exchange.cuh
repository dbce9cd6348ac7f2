// Kernels of the cross-GPU exchange of decode partials: the push of a finished partial into
// every rank's exchange buffer and the bounded wait-and-merge.  The buffer layout, the flag
// protocol and the rules after a timeout are described in pd_exchange_layout.cuh.
#pragma once

#include "pd_exchange_layout.cuh"

namespace pd {

// One CTA per destination rank: copy this rank's partial into the destination's slot for this
// rank, make it visible system-wide, then publish the flags.
__global__ void __launch_bounds__(256)
exchange_push_kernel(const float* __restrict__ local, PeerPointers peers, int world, int rank, int64_t n,
                     int units) {
  const int dst = blockIdx.x;
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(peers.buf[rank]);
  const int parity = step & 1u;
  float* out = exchange_part(peers.buf[dst], world, n, units, parity, rank);
  const int64_t n4 = n / 4;
  const float4* src4 = reinterpret_cast<const float4*>(local);
  float4* out4 = reinterpret_cast<float4*>(out);
  for (int64_t i = threadIdx.x; i < n4; i += blockDim.x) out4[i] = src4[i];
  for (int64_t i = 4 * n4 + threadIdx.x; i < n; i += blockDim.x) out[i] = local[i];
  __threadfence_system();
  __syncthreads();
  for (int u = threadIdx.x; u < units; u += blockDim.x)
    store_release_sys(exchange_flag(peers.buf[dst], world, units, parity, rank, u), step + 1u);
}

struct ExchangeMergeParams {
  unsigned char* buf;  // this rank's exchange buffer
  int32_t world, rows, d, rows_per_batch, rows_per_flag;
  void* out;
  int64_t dst_sb, dst_sh;
  float* res_o;
  float* res_lse;
  uint32_t* status;
  unsigned long long wait_ns;
  int32_t after_primary;  // launched as a programmatic dependent: order the exit after the primary grid
};

// One CTA per row (request x query head): wait (bounded) until every rank's rows of this
// step have landed here, merge them, and let the last CTA advance the step.
template <bool IO_BF16>
__global__ void __launch_bounds__(128) exchange_merge_kernel(const ExchangeMergeParams p) {
  __shared__ int ok;
  uint32_t* header = reinterpret_cast<uint32_t*>(p.buf);
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(header);
  const int parity = step & 1u;
  const int64_t n = (int64_t)p.rows * (p.d + 1);
  const int units = p.rows / p.rows_per_flag;
  const int row = blockIdx.x;
  if (threadIdx.x == 0) {
    int good = 1;
    unsigned long long t0 = 0;
    for (int r = 0; r < p.world && good; ++r) {
      const uint32_t* flag = exchange_flag(p.buf, p.world, units, parity, r, row / p.rows_per_flag);
      unsigned spins = 0;
      for (;;) {
        if (load_acquire_sys(flag) == step + 1u) break;
        if ((++spins & 15u) == 0) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (t0 == 0) t0 = now;
          if (now - t0 > p.wait_ns) {
            if (p.status) atomicOr(p.status, PD_DEV_TIMEOUT);
            good = 0;
            break;
          }
        }
        __nanosleep(100);
      }
    }
    ok = good;
  }
  __syncthreads();
  if (ok) {
    float m = -INFINITY;
    for (int r = 0; r < p.world; ++r)
      m = fmaxf(m, __ldcg(exchange_part(p.buf, p.world, n, units, parity, r) + (int64_t)p.rows * p.d + row));
    float denom = 0.f;
    if (m > -INFINITY)
      for (int r = 0; r < p.world; ++r) {
        const float lse = __ldcg(exchange_part(p.buf, p.world, n, units, parity, r) + (int64_t)p.rows * p.d + row);
        if (lse > -INFINITY) denom += exp2f(lse - m);
      }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    const int64_t dst = (int64_t)(row / p.rows_per_batch) * p.dst_sb + (int64_t)(row % p.rows_per_batch) * p.dst_sh;
    for (int d = threadIdx.x; d < p.d; d += blockDim.x) {
      float acc = 0.f;
      if (denom > 0.f)
        for (int r = 0; r < p.world; ++r) {
          const float* part = exchange_part(p.buf, p.world, n, units, parity, r);
          const float lse = __ldcg(part + (int64_t)p.rows * p.d + row);
          if (lse > -INFINITY) acc += exp2f(lse - m) * __ldcg(part + (int64_t)row * p.d + d);
        }
      const float o = acc * inv;
      if (p.out) io_store<IO_BF16>(p.out, dst + d, o);
      if (p.res_o) p.res_o[(int64_t)row * p.d + d] = o;
    }
    if (threadIdx.x == 0 && p.res_lse) p.res_lse[row] = denom > 0.f ? m + log2f(denom) : -INFINITY;
  }
  // A merge launched ahead of the end of the decode kernel (programmatic dependent launch) never
  // needs that kernel's completion for its data (the flags say what has arrived), but it must
  // not finish before it: the stream's next kernel waits only for this one.
  if (p.after_primary) asm volatile("griddepcontrol.wait;" ::: "memory");
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
