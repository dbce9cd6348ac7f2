// Layout of the exchange buffers (shared by the exchange kernels and the streaming decode kernel)
// of the cross-GPU exchange of decode partials without a collective library: every rank stores its
// partial straight into every peer's exchange buffer over NVLink (plain peer stores, no
// multicast, no loads from peer memory), raises flags there, and each rank merges what has
// landed in its own memory.  Used by the KV-range-sharded long-context path in place of
// all-gather + merge; the arithmetic is the log-sum-exp merge of
// pagedattn/triton_decode.py:221-240 over ranks instead of splits.
//
// Two producers fill the buffers: exchange_push_kernel copies a finished partial (any decode
// kernel made it), and the streaming decode kernel can store each (request, kv head) unit's
// rows itself the moment its own merge of that unit is done (PushTargets), so that no push
// launch exists and a unit's rows cross NVLink while other units are still being decoded.
//
// Exchange buffer of one rank (identical layout on every rank; `n` = floats of one partial:
// rows * D normalised fp32 results followed by rows base-2 log-sum-exps; `units` = flags per
// partial, one per rows_per_flag consecutive rows):
//   [0]   uint32 step          steps this rank has merged
//   [1]   uint32 done_ticket   CTAs of the running merge that have finished
//   byte 256 + ((parity * world + r) * units_pad + u) * 4:  uint32 flag, step + 1 once rows
//         [u * rows_per_flag, (u + 1) * rows_per_flag) of rank r's partial of that step are here
//         (units_pad = units rounded up to 64, so every rank's flags start a 256-byte line)
//   then, 256-byte aligned, (parity * world + r) * slot * 4:  rank r's partial, slot = n rounded
//         up to a multiple of four floats so that every partial starts on a 16-byte boundary
//         (the push copies with 16-byte stores; n = rows * (D + 1) is odd-sized for most shapes)
// Two parities because a peer may run one step ahead of this rank, never two: its next push
// needs its own merge of this step, which needs this rank's flags of this step.
//
// Every wait is bounded (one second unless the caller asks for less): on expiry the kernel sets
// PD_DEV_TIMEOUT in the status word, skips the merge and returns.  Ranks that gave up and ranks
// that did not may then disagree about flag values, so after PD_DEV_TIMEOUT every rank's
// buffer has to be zero-filled again before the next step.
#pragma once

#include "pd_common.cuh"

namespace pd {

constexpr int kMaxRanks = 16;
constexpr int kExchangeHeaderBytes = 256;
constexpr unsigned long long kExchangeWaitNs = 1000000000ull;

struct PeerPointers {
  unsigned char* buf[kMaxRanks];
};

// Floats from one partial's slot to the next: n rounded up to a whole number of 16-byte units.
__host__ __device__ inline int64_t exchange_slot_floats(int64_t n) { return (n + 3) & ~(int64_t)3; }
__host__ __device__ inline int64_t exchange_units_pad(int64_t units) { return (units + 63) & ~(int64_t)63; }

// Byte offset of the flag of unit u of rank r's partial of the given parity.
__host__ __device__ inline uint64_t exchange_flag_offset(int world, int64_t units, int parity, int r, int64_t u) {
  return kExchangeHeaderBytes + (uint64_t)(((int64_t)parity * world + r) * exchange_units_pad(units) + u) * 4;
}
// Byte offset of rank r's partial of the given parity inside an exchange buffer.
__host__ __device__ inline uint64_t exchange_part_offset(int world, int64_t n, int64_t units, int parity, int r) {
  return kExchangeHeaderBytes + (uint64_t)2 * world * exchange_units_pad(units) * 4 +
         (uint64_t)((int64_t)parity * world + r) * exchange_slot_floats(n) * 4;
}
__host__ __device__ inline uint64_t exchange_bytes(int world, int64_t n, int64_t units) {
  return exchange_part_offset(world, n, units, 1, world - 1) + (uint64_t)exchange_slot_floats(n) * 4;
}

__device__ __forceinline__ uint32_t* exchange_flag(unsigned char* buf, int world, int64_t units, int parity, int r,
                                                   int64_t u) {
  return reinterpret_cast<uint32_t*>(buf + exchange_flag_offset(world, units, parity, r, u));
}
__device__ __forceinline__ float* exchange_part(unsigned char* buf, int world, int64_t n, int64_t units, int parity,
                                                int r) {
  return reinterpret_cast<float*>(buf + exchange_part_offset(world, n, units, parity, r));
}
__device__ __forceinline__ void store_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// What the streaming decode kernel needs to deliver its final rows itself: every rank's
// exchange buffer, and the shape of the partial (world == 0: no exchange, the kernel writes
// its results where Params says).
struct PushTargets {
  PeerPointers peers;
  int32_t world, rank;
  int32_t rows, units;  // rows = batch * num_q_heads; units = batch * num_kv_heads
};

}  // namespace pd
