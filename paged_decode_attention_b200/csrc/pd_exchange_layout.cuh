// Layout of the exchange buffers (shared by the exchange kernels and the streaming decode kernel)
// of the cross-GPU exchange of decode partials without a collective library: every rank stores
// its partial straight into every peer's exchange buffer over NVLink (plain peer stores, no
// multicast, no loads from peer memory) and each rank merges what has landed in its own memory.
// Used by the KV-range-sharded long-context path in place of all-gather + merge; the arithmetic
// is the log-sum-exp merge of pagedattn/triton_decode.py:221-240 over ranks instead of splits.
//
// Two producers fill the buffers: exchange_push_kernel copies a finished partial (any decode
// kernel made it), and the streaming decode kernel can store each (request, kv head) unit's
// rows itself the moment its own merge of that unit is done (PushTargets), so that no push
// launch exists and a unit's rows cross NVLink while other units are still being decoded.
//
// Every value travels as one 8-byte word that carries its own arrival mark: the float's bits in
// the low half and the step's mark (step + 1, never 0) in the high half.  An aligned 8-byte
// store is indivisible, so a reader that finds the mark it waits for has the value too: no
// fence on the sending side, no separate flag, no acquire on the receiving side, and the data
// is usable one NVLink crossing after it was produced.  (The price, twice the bytes, is nothing
// here: a partial is tens of kilobytes.)
//
// Exchange buffer of one rank (identical layout on every rank; rows = batch * query heads):
//   [0]   uint32 step          steps this rank has merged
//   [1]   uint32 done_ticket   CTAs of the running merge that have finished
//   byte 256 + (parity * world + r) * slot:  rank r's partial of the steps of that parity,
//         slot = (rows * D + rows) words of 8 bytes, rounded up to 256 bytes:
//         word row * D + d       = normalised fp32 result (row, d)
//         word rows * D + row    = base-2 log-sum-exp of the row (-inf for an empty partial)
// Two parities because a peer may run one step ahead of this rank, never two: its next push
// needs its own merge of this step, which needs this rank's words of this step.  A slot is
// therefore rewritten two steps later, with another mark; stale words never match.
//
// Every wait is bounded (one second unless the caller asks for less): on expiry the kernel sets
// PD_DEV_TIMEOUT in the status word, skips what it could not merge and returns.  Ranks that
// gave up and ranks that did not may then disagree about the step, so after PD_DEV_TIMEOUT
// every rank's buffer has to be zero-filled again before the next step.
#pragma once

#include "pd_common.cuh"

namespace pd {

constexpr int kMaxRanks = 16;
constexpr int kExchangeHeaderBytes = 256;
constexpr unsigned long long kExchangeWaitNs = 1000000000ull;

struct PeerPointers {
  unsigned char* buf[kMaxRanks];
};

// Bytes from one partial's slot to the next.
__host__ __device__ inline uint64_t exchange_slot_bytes(int64_t rows, int d) {
  return ((uint64_t)rows * (d + 1) * 8 + 255) & ~(uint64_t)255;
}
// Byte offset of rank r's partial of the given parity inside an exchange buffer.
__host__ __device__ inline uint64_t exchange_part_offset(int world, int64_t rows, int d, int parity, int r) {
  return kExchangeHeaderBytes + (uint64_t)((int64_t)parity * world + r) * exchange_slot_bytes(rows, d);
}
__host__ __device__ inline uint64_t exchange_bytes(int world, int64_t rows, int d) {
  return kExchangeHeaderBytes + (uint64_t)2 * world * exchange_slot_bytes(rows, d);
}

__device__ __forceinline__ unsigned long long* exchange_part(unsigned char* buf, int world, int64_t rows, int d,
                                                             int parity, int r) {
  return reinterpret_cast<unsigned long long*>(buf + exchange_part_offset(world, rows, d, parity, r));
}
// A value and its arrival mark in one word.
__device__ __forceinline__ unsigned long long marked(float x, uint32_t mark) {
  return ((unsigned long long)mark << 32) | (unsigned long long)__float_as_uint(x);
}
// Indivisible stores of one and of two marked words (the pair 16-byte aligned).
__device__ __forceinline__ void store_marked(unsigned long long* addr, float x, uint32_t mark) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(addr), "l"(marked(x, mark)) : "memory");
}
__device__ __forceinline__ void store_marked2(unsigned long long* addr, float x0, float x1, uint32_t mark) {
  asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(addr), "l"(marked(x0, mark)), "l"(marked(x1, mark))
               : "memory");
}
__device__ __forceinline__ unsigned long long load_marked(const unsigned long long* addr) {
  unsigned long long w;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(addr) : "memory");
  return w;
}

// What the streaming decode kernel needs to deliver its final rows itself: every rank's
// exchange buffer, and the shape of the partial (world == 0: no exchange, the kernel writes
// its results where Params says).
struct PushTargets {
  PeerPointers peers;
  int32_t world, rank;
  int32_t rows;  // batch * num_q_heads
};

}  // namespace pd
