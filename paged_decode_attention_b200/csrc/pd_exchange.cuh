// Kernels of the cross-GPU exchange of decode partials: the push of a finished partial into
// every rank's exchange buffer and the bounded wait-and-merge.  The buffer layout, the marked
// words and the rules after a timeout are described in pd_exchange_layout.cuh.
#pragma once

#include "pd_exchange_layout.cuh"

namespace pd {

// One CTA per destination rank: this rank's partial (rows * D results, then rows log-sum-exps)
// goes into the destination's slot for this rank, every float as a marked word.  No fence and
// no flag: each word announces itself.
__global__ void __launch_bounds__(256)
exchange_push_kernel(const float* __restrict__ local, PeerPointers peers, int world, int rank, int rows, int d) {
  const int dst = blockIdx.x;
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(peers.buf[rank]);
  unsigned long long* out = exchange_part(peers.buf[dst], world, rows, d, step & 1u, rank);
  const int64_t n = (int64_t)rows * (d + 1);  // the flat partial has exactly the slot's word order
  const int64_t n2 = n / 2;
  for (int64_t i = threadIdx.x; i < n2; i += blockDim.x) store_marked2(out + 2 * i, local[2 * i], local[2 * i + 1], step + 1u);
  if ((n & 1) && threadIdx.x == 0) store_marked(out + n - 1, local[n - 1], step + 1u);
}

struct ExchangeMergeParams {
  unsigned char* buf;  // this rank's exchange buffer
  int32_t world, rows, d, rows_per_batch;
  void* out;
  int64_t dst_sb, dst_sh;
  float* res_o;
  float* res_lse;
  uint32_t* status;
  unsigned long long wait_ns;
  int32_t after_primary;  // launched as a programmatic dependent: order the exit after the primary grid
};

// Waits (bounded) for the word at `addr` to carry `mark`; false when the wait gave up.
__device__ __forceinline__ bool await_marked(const unsigned long long* addr, uint32_t mark, unsigned long long wait_ns,
                                             unsigned long long& t0, float& x) {
  unsigned spins = 0;
  for (;;) {
    const unsigned long long w = load_marked(addr);
    if ((uint32_t)(w >> 32) == mark) {
      x = __uint_as_float((uint32_t)w);
      return true;
    }
    if ((++spins & 15u) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      if (now - t0 > wait_ns) return false;
    }
    __nanosleep(100);
  }
}

// One CTA per row (request x query head).  Thread r < world first waits (bounded) for rank r's
// log-sum-exp of the row - the word a rank writes for a row once its data words are on their way -
// so that during a long wait (the decode kernel may still be running: see after_primary) only
// `world` threads of the CTA poll; then one thread per head_dim column collects its words (by
// then a short wait at most) and merges them.  The last CTA advances the step.
template <bool IO_BF16>
__global__ void __launch_bounds__(128) exchange_merge_kernel(const ExchangeMergeParams p) {
  __shared__ float s_lse[kMaxRanks];
  __shared__ int s_bad;
  uint32_t* header = reinterpret_cast<uint32_t*>(p.buf);
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(header);
  const int parity = step & 1u;
  const uint32_t mark = step + 1u;
  const int row = blockIdx.x;
  unsigned long long t0 = 0;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const unsigned long long* part = exchange_part(p.buf, p.world, p.rows, p.d, parity, threadIdx.x);
    float x = -INFINITY;
    if (!await_marked(part + (int64_t)p.rows * p.d + row, mark, p.wait_ns, t0, x)) s_bad = 1;
    s_lse[threadIdx.x] = x;
  }
  __syncthreads();
  bool ok = s_bad == 0;
  float m = -INFINITY, denom = 0.f;
  if (ok) {
    for (int r = 0; r < p.world; ++r) m = fmaxf(m, s_lse[r]);
    if (m > -INFINITY)
      for (int r = 0; r < p.world; ++r)
        if (s_lse[r] > -INFINITY) denom += exp2f(s_lse[r] - m);
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  const int64_t dst = (int64_t)(row / p.rows_per_batch) * p.dst_sb + (int64_t)(row % p.rows_per_batch) * p.dst_sh;
  for (int d = threadIdx.x; d < p.d && ok; d += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < p.world && ok; ++r) {
      const unsigned long long* part = exchange_part(p.buf, p.world, p.rows, p.d, parity, r);
      float x;
      ok = await_marked(part + (int64_t)row * p.d + d, mark, p.wait_ns, t0, x);
      if (denom > 0.f && s_lse[r] > -INFINITY) acc += exp2f(s_lse[r] - m) * x;
    }
    if (!ok) break;
    const float o = acc * inv;
    if (p.out) io_store<IO_BF16>(p.out, dst + d, o);
    if (p.res_o) p.res_o[(int64_t)row * p.d + d] = o;
  }
  if (ok && threadIdx.x == 0 && p.res_lse) p.res_lse[row] = denom > 0.f ? m + log2f(denom) : -INFINITY;
  if (!ok && p.status) atomicOr(p.status, PD_DEV_TIMEOUT);
  // A merge launched ahead of the end of the decode kernel (programmatic dependent launch) never
  // needs that kernel's completion for its data (the words say what has arrived), but it must
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
