// Streaming decode kernel for sm_100a: a persistent grid of one CTA per SM.
//
// Work decomposition.  Every request's KV range (or every explicit split of it) for one block
// of HB kv heads is a "virtual sequence" of 16-token tiles.  All virtual sequences are laid end
// to end and the tile sequence is cut into equal contiguous shares, one per worker.  A worker
// is HB consumer warps (one per kv head of the block) plus one producer warp; a CTA hosts
// 8/HB workers (at most 4).  Shares are balanced to one tile whatever the length distribution,
// and they are derived on the device from seq_lens, so the host never synchronises.
//
// Data movement.  The producer warp resolves each tile's page through the block table (32
// tiles' entries are fetched with one coalesced load ahead of use) and issues tiled TMA loads
// (cp.async.bulk.tensor) of the K and V boxes [HB heads][16 tokens][128 B] with the 128-byte
// swizzle into a ring of shared-memory stages; completion is tracked by mbarriers
// (full/empty per stage).  Per-(token, head) scales ride along as untiled bulk copies.  The
// ring runs across request boundaries, so HBM requests never drain between requests.
//
// Math.  Each consumer warp keeps the (padded to 16) query rows of its group as mma A
// fragments in registers, computes S = Q K^T with mma.sync m16n8k16 (K rows via ldmatrix, or
// 16-byte shared loads plus in-register e5m2 -> f16 conversion; int8 keys run unconverted on
// the integer path, m16n8k32, against the query split into two int8 digits), applies a base-2
// online softmax with warp shuffles (the reference's recurrence,
// pagedattn/triton_decode.py:159-166), and accumulates O += P V in fp32.  Scales factor out of
// both contractions: S is multiplied by the K scale per token, P by the V scale per token, so
// 8-bit pages are only ever converted, never multiplied element-wise.  Where the ring holds five
// stages or more (8-bit shapes) a warp takes two tiles per softmax step.
//
// Results.  A (worker, virtual sequence) segment that covers a whole unsplit request writes
// its output row directly; any other segment writes a normalised fp32 partial plus its base-2
// log-sum-exp into slot (worker + virtual sequence) of the scratch and takes a ticket on the
// (request, kv head) counter; the warp whose ticket completes the count merges the request's
// slots in place (pagedattn/triton_decode.py:221-240).  No second kernel, and no warp ever
// waits for another.  Every counter is back at zero when the kernel ends.  In pushing mode
// (KV-range sharding over several GPUs) every unit takes the merge path, and the merging warp
// also stores the unit's rows into every rank's exchange buffer (pd_exchange_layout.cuh).
//
// Every wait is bounded: a wait that exceeds its limit sets PD_DEV_TIMEOUT in the status word,
// raises the CTA's abort flag, and all warps leave their loops; the producer then waits (again
// bounded) for the copies it still has in flight before the CTA exits.
#pragma once

#include <cuda.h>

#include "pd_common.cuh"
#include "pd_exchange_layout.cuh"

namespace pd {

// ---------------------------------------------------------------------------------------------
// configuration
// ---------------------------------------------------------------------------------------------
constexpr int kTileTokens = 16;

// 16-bit page element types: both are moved and multiplied as they are
__host__ __device__ constexpr bool is_16bit(int kv) { return kv == PD_KV_F16 || kv == PD_KV_BF16; }
constexpr int kMaxVseq = 4096;
constexpr int kMinTilesPerWorker = 4;
constexpr int kMergeRadix = 8;
constexpr int kWholeTiles = 16;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kMaxStages = 12;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

// Workers per CTA: eight consumer warps' worth (at most four workers).
__host__ __device__ constexpr int base_workers_per_cta(int hb) { return 8 / hb < 4 ? 8 / hb : 4; }

template <int KV, int D, int HB, bool SCALED>
struct StreamCfg {
  static constexpr int EB = is_16bit(KV) ? 2 : 1;
  static constexpr int ROWB = D * EB;
  static_assert(ROWB == 64 || ROWB == 128 || ROWB == 256 || ROWB == 512,
                "a row is 64 bytes or 1, 2 or 4 pieces of 128 bytes");
  static constexpr int PITCH = ROWB < 128 ? ROWB : 128;     // bytes of one shared-memory row
  static constexpr int CPR = PITCH / 16;                    // 16-byte chunks per shared-memory row
  static constexpr int NC = ROWB / PITCH;                   // pieces (TMA boxes) per row
  static constexpr int BOX_ELEMS = PITCH / EB;              // elements of one piece
  static constexpr int WARPS_PER_WORKER = HB + 1;
  static constexpr int CHUNK_BYTES = HB * kTileTokens * PITCH; // one TMA box
  static constexpr int TILE_BYTES = NC * CHUNK_BYTES;        // K (or V) of one tile
  static constexpr int SCALE_BYTES = SCALED ? 2048 : 0;      // K scales at +0, V scales at +1024
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES + SCALE_BYTES;
  static constexpr int KSTEPS = D / 16;
  static constexpr int MT = D / 16;                          // 16-row tiles of head_dim in O^T
};

struct StreamParams {
  Params p;
  int32_t nvseq, nhb, splits, nstage, wpc;
  uint32_t bar_off, meta_off, misc_off, prefix_off, count_off, bound_off;
  // Query staging: qstage_warp_bytes > 0 when the query rows of one kv head's group are one dense
  // run in q and shared memory has room; every consumer warp then owns that many bytes at
  // qstage_off, rows at a pitch of head_dim * 2 + 16 bytes (the 16 spread the rows over the banks).
  uint32_t qstage_off, qstage_warp_bytes;
  int32_t seg_cost;  // tiles' worth of time that one segment end costs a worker (0: shares of equal tile counts)
  int32_t* tickets;  // one arrival counter per (request, kv head), zero when the kernel starts
  uint32_t scale_tx_bytes;  // bytes of one scale copy: 16 tokens * Hkv * 2
  // KV-range-sharded runs: where every finished (request, kv head) unit is also stored, on every
  // rank of the group (push.world == 0 otherwise).  Every unit then goes through the in-kernel
  // merge, which is the one place that delivers final rows.
  PushTargets push;
};

// Where the TMA swizzle puts 16-byte chunk `chunk` of token row `token`: the 128-byte mode
// XORs the chunk index with the row index mod 8, the 64-byte mode (64-byte rows, four chunks)
// with bits 1-2 of the row index.
template <int PITCH>
__device__ __forceinline__ int swizzled_chunk(int chunk, int token) {
  if constexpr (PITCH == 128) return chunk ^ (token & 7);
  else return chunk ^ ((token >> 1) & 3);
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Waits for a barrier phase for at most kWaitLimitNs.  Returns false (after raising the CTA's
// abort flag and PD_DEV_TIMEOUT) when it gives up or when another warp already aborted.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, uint32_t* status,
                                            volatile int* abort_flag, bool heed_abort,
                                            unsigned long long limit_ns = kWaitLimitNs) {
  const unsigned long long t0 = global_timer_ns();
  unsigned spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (heed_abort && *abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        if (status) atomicOr(status, PD_DEV_TIMEOUT);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t* status,
                                          volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, status, abort_flag, true);
}

// Tiled TMA load of one 4-D box into shared memory; completion is counted on `bar`.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"((unsigned long long)src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void lds128(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void lds64(uint32_t addr, uint32_t (&r)[2]) {
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t r;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(addr));
  return r;
}
__device__ __forceinline__ float lds_half(uint32_t addr) {
  unsigned short h;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
  return __half2float(__ushort_as_half(h));
}
// D(16x8, f32) += A(16x16, f16) * B(16x8, f16)
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// the same with bf16 inputs
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// bf16 pages are multiplied as bf16 (q, P and the output are bf16 too); every other page type
// reaches the tensor core as f16
template <int KV>
__device__ __forceinline__ void mma_kv(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (KV == PD_KV_BF16) mma_bf16(c, a, b0, b1);
  else mma_f16(c, a, b0, b1);
}
// D (16x8, s32) += A (16x32, s8, row) * B (32x8, s8, col)
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Two floats -> packed 16-bit pair in the type q and out use (bf16 with bf16 pages, else f16).
template <int KV>
__device__ __forceinline__ uint32_t pack_io2(float lo, float hi) {
  if constexpr (KV == PD_KV_BF16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else {
    return pack_half2(lo, hi);
  }
}
template <int KV>
__device__ __forceinline__ void store_io(void* row, int col, float x) {
  if constexpr (KV == PD_KV_BF16) ((__nv_bfloat16*)row)[col] = __float2bfloat16_rn(x);
  else ((__half*)row)[col] = __float2half_rn(x);
}

// Two stored 8-bit elements (bytes `lo_sel`, `lo_sel + 1` of w) -> packed f16x2, exactly.
template <int KV>
__device__ __forceinline__ uint32_t cvt_pair(uint32_t w, bool upper) {
  if constexpr (KV == PD_KV_E5M2) {
    // e5m2 is the high byte of an f16: place each byte above a zero byte
    return __byte_perm(w, 0u, upper ? 0x3424u : 0x1404u);
  } else {
    // int8: w already holds x ^ 0x80 (= x + 128 as unsigned); 0x6400 | u is the f16 1024 + u,
    // so subtracting 1152 leaves x
    const uint32_t h = __byte_perm(w, 0x64646464u, upper ? 0x4342u : 0x4140u);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h),
                              __half2half2(__ushort_as_half((unsigned short)0x6480)));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}

// ---------------------------------------------------------------------------------------------
// schedule helpers (shared by producer, consumers and the merge kernel)
// ---------------------------------------------------------------------------------------------
struct VseqInfo {
  int hb, b, split, lo, hi;
};

__device__ __forceinline__ VseqInfo vseq_info(const StreamParams& sp, int v) {
  VseqInfo i;
  i.split = v % sp.splits;
  const int t = v / sp.splits;
  i.b = t % sp.p.batch;
  i.hb = t / sp.p.batch;
  split_range(clamp_len(sp.p, i.b), i.split, sp.splits, sp.p.block_n, i.lo, i.hi);
  return i;
}

// Largest v in [0, n) with prefix[v] <= g (prefix is non-decreasing, prefix[0] = 0, g < prefix[n]).
__device__ __forceinline__ int find_vseq(const int* prefix, int n, int g) {
  int lo = 0, hi = n;  // invariant: prefix[lo] <= g < prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= g) lo = mid;
    else hi = mid;
  }
  return lo;
}

// int8 pair -> f16x2 holding 1152 + x (w is x ^ 0x80 per byte): one prmt, no subtraction.
__device__ __forceinline__ uint32_t cvt_pair_biased(uint32_t w, bool upper) {
  return __byte_perm(w, 0x64646464u, upper ? 0x4342u : 0x4140u);
}
// Transposes an 8x8 matrix of 16-bit elements held one row-pair per thread (ldmatrix layout).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// One 16-token tile of one kv head for one consumer warp.  The products are taken with the
// tokens on the M axis of the mma and the query heads of the group on its N axis ("swapped"):
//   S^T[16 tokens x 8 heads] = K[16 x D] * Q^T,   O^T[D x 8 heads] += V^T[D x 16] * P^T
// so a group of up to 8 heads fills the 8-wide N dimension instead of padding a 16-row M
// (NG = 2 covers groups of 9..16).  Thread (g = lane / 4, t = lane % 4) owns tokens g and g + 8
// of S^T and heads 2t, 2t + 1 (+ 8 per n-tile), the same heads it owns in O^T, so the softmax
// state (m, l) stays in the thread; P^T reaches the B-operand layout with two movmatrix.
// `kbase` is the warp's K rows in the stage (V follows at TILE_BYTES), `scales` the address of
// this head's K scale of token 0 (V scales 1024 bytes further, token pitch hkv * 2).
// MASKED: the last tile holds fewer than 16 live tokens (`valid`); full tiles skip every mask.
// NT = 2 takes two consecutive tiles of the same request (two stages) as one 32-token softmax
// step: one running-maximum update, one rescale, and two independent score chains in flight.
template <int KV, int D, int HB, bool SCALED, int NG, bool MASKED, int NT = 1>
__device__ __forceinline__ void consume_tile(
    const uint32_t (&kbase)[NT], const uint32_t (&scales)[NT], const int hkv, const int valid,
    const float scale_log2, const int lane,
    const uint32_t (&qb)[StreamCfg<KV, D, HB, SCALED>::KSTEPS][NG][2], const float (&qstep)[NG][2],
    float (&m)[NG][2], float (&l)[NG][2], float (&o)[StreamCfg<KV, D, HB, SCALED>::MT][NG][4],
    float (&psum)[NG][4]) {
  using C = StreamCfg<KV, D, HB, SCALED>;
  constexpr unsigned kFull = 0xffffffffu;
  const int gq = lane >> 2, tq = lane & 3;

  // ---- S^T = K Q^T ------------------------------------------------------------------------------
  // Two accumulators per n-tile keep two dependent chains in flight: one per tile when NT = 2,
  // else one for the even and one for the odd k-steps (summed below).
  float s[2][NG][4];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) s[u][ng][0] = s[u][ng][1] = s[u][ng][2] = s[u][ng][3] = 0.f;
  }
  if constexpr (is_16bit(KV)) {
    // A fragments by ldmatrix: matrices (tokens 0-7, lo), (8-15, lo), (0-7, hi), (8-15, hi) where
    // lo/hi are the two 16-byte chunks of the k-step
    const int mi = lane >> 3;
    const int token = 8 * (mi & 1) + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < C::KSTEPS; ++ks) {
      const int chunk = ((2 * ks) % C::CPR) + (mi >> 1);
      const uint32_t off = token * C::PITCH + ((2 * ks) / C::CPR) * C::CHUNK_BYTES +
                           (swizzled_chunk<C::PITCH>(chunk, token) << 4);
#pragma unroll
      for (int u = 0; u < NT; ++u) {
        uint32_t a[4];
        ldmatrix_x4(kbase[u] + off, a);
#pragma unroll
        for (int ng = 0; ng < NG; ++ng)
          mma_kv<KV>(s[NT == 2 ? u : (ks & 1)][ng], a, qb[ks][ng][0], qb[ks][ng][1]);
      }
    }
  } else {
    // tokens g and g + 8 share the swizzle phase; a thread reads CPT = 2 (128-byte pieces) or 1
    // (64-byte rows) of the 16-byte chunks of each piece c of the row, chunk CPT*t + jh; word i
    // of the cj-th chunk it reads feeds k-step 4*cj + i
    constexpr int CPT = C::CPR / 4;
    int s_hi[NT][NG][4], s_lo[NT][NG][4];  // int8 only: the two digits are independent chains
#pragma unroll
    for (int u = 0; u < NT; ++u) {
#pragma unroll
      for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
        for (int r = 0; r < 4; ++r) s_hi[u][ng][r] = s_lo[u][ng][r] = 0;
      }
    }
#pragma unroll
    for (int cj = 0; cj < CPT * C::NC; ++cj) {
      const int c = cj / CPT, jh = cj % CPT;
      const uint32_t ch = gq * C::PITCH + (uint32_t)c * C::CHUNK_BYTES +
                          ((uint32_t)swizzled_chunk<C::PITCH>(CPT * tq + jh, gq) << 4);
#pragma unroll
      for (int u = 0; u < NT; ++u) {
        uint32_t w0[4], w1[4];
        lds128(kbase[u] + ch, w0);
        lds128(kbase[u] + ch + 8 * C::PITCH, w1);
        if constexpr (KV == PD_KV_I8) {
          // int8 keys go to the integer tensor-core path as they are: words 2*m2 and 2*m2 + 1
          // of the chunk are the two k halves of one m16n8k32 step, against the query's high
          // and low int8 digits (qb[.][.][0] and [1], see the prologue); no conversions
#pragma unroll
          for (int m2 = 0; m2 < 2; ++m2) {
            const uint32_t a[4] = {w0[2 * m2], w1[2 * m2], w0[2 * m2 + 1], w1[2 * m2 + 1]};
            const int ks = 4 * cj + 2 * m2;
#pragma unroll
            for (int ng = 0; ng < NG; ++ng) {
              mma_s8(s_hi[u][ng], a, qb[ks][ng][0], qb[ks + 1][ng][0]);
              mma_s8(s_lo[u][ng], a, qb[ks][ng][1], qb[ks + 1][ng][1]);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t a[4];
            a[0] = cvt_pair<KV>(w0[i], false);
            a[1] = cvt_pair<KV>(w1[i], false);
            a[2] = cvt_pair<KV>(w0[i], true);
            a[3] = cvt_pair<KV>(w1[i], true);
#pragma unroll
            for (int ng = 0; ng < NG; ++ng)
              mma_kv<KV>(s[NT == 2 ? u : (i & 1)][ng], a, qb[4 * cj + i][ng][0], qb[4 * cj + i][ng][1]);
          }
        }
      }
    }
    if constexpr (KV == PD_KV_I8) {
      // exact integer dot products with the two digits; the query's step size comes in below
#pragma unroll
      for (int u = 0; u < NT; ++u) {
#pragma unroll
        for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
          for (int r = 0; r < 4; ++r) s[u][ng][r] = (float)(s_hi[u][ng][r] * 128 + s_lo[u][ng][r]);
        }
      }
    }
  }
  if constexpr (NT == 1 && KV != PD_KV_I8) {
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
      for (int r = 0; r < 4; ++r) s[0][ng][r] += s[1][ng][r];
    }
  }

  // ---- scale, mask, online softmax; P^T into B-operand layout ---------------------------------
  float f[NT][2], vs[NT][2];  // score factors and V scales (times 256) of tokens g and g + 8
#pragma unroll
  for (int u = 0; u < NT; ++u) {
    f[u][0] = f[u][1] = scale_log2;
    vs[u][0] = vs[u][1] = 1.f;
    if constexpr (SCALED) {
      const uint32_t sa = scales[u] + gq * hkv * 2;
      f[u][0] *= lds_half(sa);
      f[u][1] *= lds_half(sa + 8 * hkv * 2);
      vs[u][0] = lds_half(sa + 1024) * 256.f;
      vs[u][1] = lds_half(sa + 1024 + 8 * hkv * 2) * 256.f;
    }
  }
  uint32_t pb[NT][NG][2];
  float alpha[NG][2];
  bool moved = false;
#pragma unroll
  for (int ng = 0; ng < NG; ++ng) {
    float x[NT][4];
    float mx0 = -INFINITY, mx1 = -INFINITY;  // heads 2t, 2t+1 over the thread's tokens
#pragma unroll
    for (int u = 0; u < NT; ++u) {
#pragma unroll
      for (int r = 0; r < 4; ++r) x[u][r] = s[u][ng][r];
      if constexpr (KV == PD_KV_I8) {  // the quantisation step of the query rows of heads 2t, 2t+1
        x[u][0] *= qstep[ng][0];
        x[u][1] *= qstep[ng][1];
        x[u][2] *= qstep[ng][0];
        x[u][3] *= qstep[ng][1];
      }
      x[u][0] *= f[u][0];
      x[u][1] *= f[u][0];
      x[u][2] *= f[u][1];
      x[u][3] *= f[u][1];
      if constexpr (MASKED) {
        if (u == NT - 1) {
          if (gq >= valid) x[u][0] = x[u][1] = -INFINITY;
          if (gq + 8 >= valid) x[u][2] = x[u][3] = -INFINITY;
        }
      }
      mx0 = fmaxf(mx0, fmaxf(x[u][0], x[u][2]));
      mx1 = fmaxf(mx1, fmaxf(x[u][1], x[u][3]));
    }
#pragma unroll
    for (int sh = 4; sh < 32; sh <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, sh));
      mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, sh));
    }
    const float mn0 = fmaxf(m[ng][0], mx0), mn1 = fmaxf(m[ng][1], mx1);  // finite: token 0 is live
    alpha[ng][0] = fast_exp2(m[ng][0] - mn0);
    alpha[ng][1] = fast_exp2(m[ng][1] - mn1);
    moved = moved || alpha[ng][0] != 1.f || alpha[ng][1] != 1.f;
    m[ng][0] = mn0;
    m[ng][1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int u = 0; u < NT; ++u) {
      const float p0 = fast_exp2(x[u][0] - mn0), p1 = fast_exp2(x[u][1] - mn1);
      const float p2 = fast_exp2(x[u][2] - mn0), p3 = fast_exp2(x[u][3] - mn1);
      sum0 += p0 + p2;
      sum1 += p1 + p3;
      // (token g | g+8, heads 2t, 2t+1) -> (tokens 2t, 2t+1 | 2t+8, 2t+9, head g)
      pb[u][ng][0] = movmatrix_trans(SCALED ? pack_io2<KV>(p0 * vs[u][0], p1 * vs[u][0]) : pack_io2<KV>(p0, p1));
      pb[u][ng][1] = movmatrix_trans(SCALED ? pack_io2<KV>(p2 * vs[u][1], p3 * vs[u][1]) : pack_io2<KV>(p2, p3));
    }
    l[ng][0] = l[ng][0] * alpha[ng][0] + sum0;
    l[ng][1] = l[ng][1] * alpha[ng][1] + sum1;
  }
  // the running maxima settle after the first tiles; skip the rescale when nobody's moved
  if (__any_sync(kFull, moved)) {
#pragma unroll
    for (int mt = 0; mt < C::MT; ++mt) {
#pragma unroll
      for (int ng = 0; ng < NG; ++ng) {
        o[mt][ng][0] *= alpha[ng][0];
        o[mt][ng][1] *= alpha[ng][1];
        o[mt][ng][2] *= alpha[ng][0];
        o[mt][ng][3] *= alpha[ng][1];
      }
    }
    if constexpr (KV == PD_KV_I8) {
#pragma unroll
      for (int ng = 0; ng < NG; ++ng) {
        psum[ng][0] *= alpha[ng][0];
        psum[ng][1] *= alpha[ng][1];
        psum[ng][2] *= alpha[ng][0];
        psum[ng][3] *= alpha[ng][1];
      }
    }
  }

  // ---- O^T += V^T P^T ---------------------------------------------------------------------------
  // Rows of V past `valid` hold whatever the page holds.  Every int8 byte is a finite number,
  // so P = 0 already removes it; f16 / e5m2 garbage may be NaN and is zeroed in masked tiles.
  constexpr bool kMaskV = MASKED && KV != PD_KV_I8;
  uint32_t keep_lo = 0xffffffffu, keep_hi = 0xffffffffu;  // tokens (2t, 2t+1), (2t+8, 2t+9)
  if constexpr (kMaskV) {
    keep_lo = (2 * tq < valid ? 0x0000ffffu : 0u) | (2 * tq + 1 < valid ? 0xffff0000u : 0u);
    keep_hi = (2 * tq + 8 < valid ? 0x0000ffffu : 0u) | (2 * tq + 9 < valid ? 0xffff0000u : 0u);
  }
#pragma unroll
  for (int u = 0; u < NT; ++u) {
    const uint32_t vbase = kbase[u] + C::TILE_BYTES;
    const bool mask_this = kMaskV && u == NT - 1;
    if constexpr (is_16bit(KV)) {
      // transposed 8x8 matrices (tokens 0-7, lo), (0-7, hi), (8-15, lo), (8-15, hi) of the 16
      // head_dim columns of m-tile mt: A rows are head_dim 16*mt + g and + 8
      const int mi = lane >> 3;
      const int token = 8 * (mi >> 1) + (lane & 7);
      const uint32_t row = vbase + token * C::PITCH;
#pragma unroll
      for (int mt = 0; mt < C::MT; ++mt) {
        const int chunk = ((2 * mt) % C::CPR) + (mi & 1);
        uint32_t a[4];
        ldmatrix_x4_trans(row + ((2 * mt) / C::CPR) * C::CHUNK_BYTES +
                              (swizzled_chunk<C::PITCH>(chunk, token) << 4), a);
        if (mask_this) {
          a[0] &= keep_lo;
          a[1] &= keep_lo;
          a[2] &= keep_hi;
          a[3] &= keep_hi;
        }
#pragma unroll
        for (int ng = 0; ng < NG; ++ng) mma_kv<KV>(o[mt][ng], a, pb[u][ng][0], pb[u][ng][1]);
      }
    } else {
      // 8-bit V: from each of its four tokens the thread reads BPT = PITCH / 8 contiguous bytes
      // of every piece c of the row (one 16- or 8-byte load) - head_dim columns c*PITCH + BPT*g
      // .. + BPT-1 - and transposes bytes in registers.  m-tile c*(PITCH/16) + 2*i + h then
      // holds column c*PITCH + BPT*g + 4*i + 2*h in its row g and the next column in its row
      // g + 8; the epilogue writes the thread's BPT columns back as one contiguous run.
      constexpr int WPT = C::PITCH / 32;  // 32-bit words per thread, token and piece
      const int tk[4] = {2 * tq, 2 * tq + 1, 2 * tq + 8, 2 * tq + 9};
#pragma unroll
      for (int c = 0; c < C::NC; ++c) {
        uint32_t r[4][WPT];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t row = vbase + c * C::CHUNK_BYTES + tk[k] * C::PITCH;
          if constexpr (C::PITCH == 128) lds128(row + (swizzled_chunk<128>(gq, tk[k]) << 4), r[k]);
          else lds64(row + (swizzled_chunk<64>(gq >> 1, tk[k]) << 4) + ((gq & 1) << 3), r[k]);
          if constexpr (KV == PD_KV_I8) {
#pragma unroll
            for (int i = 0; i < WPT; ++i) r[k][i] ^= 0x80808080u;
          }
        }
#pragma unroll
        for (int i = 0; i < WPT; ++i) {
          // bytes (c0, c2) and (c1, c3) of the token pairs side by side
          const uint32_t e01 = __byte_perm(r[0][i], r[1][i], 0x6240u), o01 = __byte_perm(r[0][i], r[1][i], 0x7351u);
          const uint32_t e23 = __byte_perm(r[2][i], r[3][i], 0x6240u), o23 = __byte_perm(r[2][i], r[3][i], 0x7351u);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int mt = c * (C::PITCH / 16) + 2 * i + h;
            uint32_t a[4];
            if constexpr (KV == PD_KV_I8) {
              // int8 values enter as 1152 + x (one prmt each); the surplus is taken out below
              a[0] = cvt_pair_biased(e01, h != 0);
              a[1] = cvt_pair_biased(o01, h != 0);
              a[2] = cvt_pair_biased(e23, h != 0);
              a[3] = cvt_pair_biased(o23, h != 0);
            } else {
              a[0] = cvt_pair<KV>(e01, h != 0);
              a[1] = cvt_pair<KV>(o01, h != 0);
              a[2] = cvt_pair<KV>(e23, h != 0);
              a[3] = cvt_pair<KV>(o23, h != 0);
            }
            if (mask_this) {
              a[0] &= keep_lo;
              a[1] &= keep_lo;
              a[2] &= keep_hi;
              a[3] &= keep_hi;
            }
#pragma unroll
            for (int ng = 0; ng < NG; ++ng) mma_kv<KV>(o[mt][ng], a, pb[u][ng][0], pb[u][ng][1]);
          }
        }
      }
    }
  }
  if constexpr (KV == PD_KV_I8) {
    // Every int8 value entered as 1152 + x.  One more mma with an all-ones A adds, in every row,
    // the sum over this call's tokens of P^T exactly as the tensor core read it to the running
    // column sums; they are rescaled with the accumulators, and 1152 times them leaves every
    // accumulator once, when the segment ends (no multiply-add per accumulator and tile).
    const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
      for (int u = 0; u < NT; ++u) mma_kv<KV>(psum[ng], ones, pb[u][ng][0], pb[u][ng][1]);
    }
  }
}

// The tile line is cut into one cell per worker: cell w holds the tiles [bound[w], bound[w + 1]).
// The cells are not equally long (a worker that crosses more request boundaries gets fewer
// tiles, see the kernel), so the cell of a tile is found by bisection over the boundaries; every
// thread derives the same boundaries from the lengths alone, which is what lets any warp count
// and find the partial results of a request.
struct CellMap {
  const int* bound;  // workers + 1 non-decreasing tile indices, bound[0] = 0, bound[workers] = total
  int workers;
  // the cell that holds tile g (0 <= g < total): the last w with bound[w] <= g
  __device__ __forceinline__ int of(int g) const {
    int lo = 0, hi = workers;  // invariant: bound[lo] <= g < bound[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (bound[mid] <= g) lo = mid;
      else hi = mid;
    }
    return lo;
  }
};

// Segments (cell, virtual sequence) that cover request b / head block hb, in the order the
// merge visits them: for every split with tiles, the cells first .. last of its tile range.
template <typename F>
__device__ __forceinline__ void for_each_segment(const int* prefix, const CellMap& cm, int v0, int splits, F&& f) {
  for (int s = 0; s < splits; ++s) {
    const int first = prefix[v0 + s], last = prefix[v0 + s + 1];
    if (last <= first) continue;
    for (int c = cm.of(first); c <= cm.of(last - 1); ++c) f(c + v0 + s);
  }
}

// Log-sum-exp merge of every partial of one (request, kv head), run by the consumer warp whose
// partial arrived last (pagedattn/triton_decode.py:221-240 for the arithmetic).  The eight
// 4-lane groups of the warp are split between rows and segments: with RP = the group size
// rounded up to a power of two (at most 8), lane group q handles row q % RP and the segments
// i with i % (8 / RP) == q / RP; a lane owns the head_dim floats 16*j + 4*c .. +3 of its row.
// Small groups thus spread a long segment list (dozens for one long-context request) over more
// lanes.  The per-phase sums are combined with shuffles.  Partials were written by other SMs:
// they are read with ld.global.cg after the ticket's fence.
template <int KV, int D>
__device__ __forceinline__ void merge_unit(const Params& p, const int* prefix, const CellMap& cm, int v0,
                                           int splits, int hg, int head_in_block, int b, int kvh,
                                           int lane, int rslot0 = 0, int rn = 0, int rstride = 1,
                                           int dst_slot = -1, const PushTargets* push = nullptr,
                                           uint32_t step = 0) {
  // Default: merge every segment the schedule gives the unit and write the final rows.  With
  // rn > 0 the inputs are instead the rn slots rslot0, rslot0 + rstride, ...; with dst_slot >= 0
  // the result goes back into that slot as a normalised partial (first level of a deep merge).
  auto for_ranges = [&](auto&& f) {
    if (rn > 0) {
      f(rslot0, rn, rstride);
      return;
    }
    for (int s = 0; s < splits; ++s) {
      const int first = prefix[v0 + s], last = prefix[v0 + s + 1];
      if (last <= first) continue;
      f(cm.of(first) + v0 + s, cm.of(last - 1) - cm.of(first) + 1, 1);
    }
  };
  constexpr int J = D / 16;
  constexpr unsigned kFull = 0xffffffffu;
  const int q = lane >> 2, c = lane & 3;
  int rp = 1;
  while (rp < p.group && rp < 8) rp <<= 1;
  const int sp_n = 8 / rp;        // segment phases
  const int phase = q / rp;
  for (int r0 = 0; r0 < p.group; r0 += 8) {
    const int row = r0 + q % rp;
    const bool live = row < p.group;
    const int64_t local = (int64_t)head_in_block * p.group + (live ? row : 0);
    // One pass with a running maximum (the partials' data loads do not wait for a first pass
    // over their log-sum-exps): when a partial raises the maximum, what has been summed so far is
    // scaled down to it.  The phases are then brought to their common maximum and added.
    float m = -INFINITY;
    float denom = 0.f;
    float acc[J][4];
#pragma unroll
    for (int j = 0; j < J; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    for_ranges([&](int slot0, int n, int stride) {
      const float* lp = p.part_lse + (int64_t)slot0 * hg + local;
      const float4* op = reinterpret_cast<const float4*>(p.part_o + ((int64_t)slot0 * hg + local) * D) + c;
#pragma unroll(J > 8 ? 1 : 2)
      for (int i = phase; i < n; i += sp_n) {
        const float lse = __ldcg(lp + (int64_t)i * stride * hg);
        float4 x[J];
#pragma unroll
        for (int j = 0; j < J; ++j) x[j] = __ldcg(op + (int64_t)i * stride * hg * (D / 4) + 4 * j);
        if (lse > m) {
          const float down = m > -INFINITY ? exp2f(m - lse) : 0.f;
          denom *= down;
#pragma unroll
          for (int j = 0; j < J; ++j) {
            acc[j][0] *= down;
            acc[j][1] *= down;
            acc[j][2] *= down;
            acc[j][3] *= down;
          }
          m = lse;
        }
        const float wgt = lse > -INFINITY ? exp2f(lse - m) : 0.f;
        denom += wgt;
#pragma unroll
        for (int j = 0; j < J; ++j) {
          acc[j][0] = fmaf(wgt, x[j].x, acc[j][0]);
          acc[j][1] = fmaf(wgt, x[j].y, acc[j][1]);
          acc[j][2] = fmaf(wgt, x[j].z, acc[j][2]);
          acc[j][3] = fmaf(wgt, x[j].w, acc[j][3]);
        }
      }
    });
    if (sp_n > 1) {
      float mall = m;
      for (int sh = 4 * rp; sh < 32; sh <<= 1) mall = fmaxf(mall, __shfl_xor_sync(kFull, mall, sh));
      const float down = m > -INFINITY ? exp2f(m - mall) : 0.f;  // mall is finite whenever m is
      denom *= down;
#pragma unroll
      for (int j = 0; j < J; ++j) {
        acc[j][0] *= down;
        acc[j][1] *= down;
        acc[j][2] *= down;
        acc[j][3] *= down;
      }
      m = mall;
    }
    for (int sh = 4 * rp; sh < 32; sh <<= 1) {
      denom += __shfl_xor_sync(kFull, denom, sh);
#pragma unroll
      for (int j = 0; j < J; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] += __shfl_xor_sync(kFull, acc[j][e], sh);
      }
    }
    if (!live || phase != 0) continue;
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    if (dst_slot >= 0) {
      // first level of a deep merge: the chunk's result replaces the partial in its first slot
      const int64_t sr = (int64_t)dst_slot * hg + local;
#pragma unroll
      for (int j = 0; j < J; ++j)
        *reinterpret_cast<float4*>(p.part_o + sr * D + 16 * j + 4 * c) =
            make_float4(acc[j][0] * inv, acc[j][1] * inv, acc[j][2] * inv, acc[j][3] * inv);
      if (c == 0) p.part_lse[sr] = denom > 0.f ? m + log2f(denom) : -INFINITY;
      continue;
    }
    const int hq = kvh * p.group + row;
    __half* dst16 = p.out ? (__half*)p.out + (int64_t)b * p.o_sb + (int64_t)hq * p.o_sh : nullptr;
    float* dst32 = p.res_o ? p.res_o + ((int64_t)b * p.hq + hq) * D : nullptr;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int col = 16 * j + 4 * c;
      const float x0 = acc[j][0] * inv, x1 = acc[j][1] * inv, x2 = acc[j][2] * inv, x3 = acc[j][3] * inv;
      if (dst16) {
        uint2 pk;
        pk.x = pack_io2<KV>(x0, x1);
        pk.y = pack_io2<KV>(x2, x3);
        *reinterpret_cast<uint2*>(dst16 + col) = pk;
      }
      if (dst32) *reinterpret_cast<float4*>(dst32 + col) = make_float4(x0, x1, x2, x3);
    }
    const float lse_out = denom > 0.f ? m + log2f(denom) : -INFINITY;
    if (p.res_o && c == 0) p.res_lse[(int64_t)b * p.hq + hq] = lse_out;
    if (push) {
      // the same row into this rank's slot of every rank's exchange buffer: plain peer stores of
      // marked words, which announce themselves (no fence, no flag)
      const int64_t grow = (int64_t)b * p.hq + hq;
      for (int r = 0; r < push->world; ++r) {
        unsigned long long* part = exchange_part(push->peers.buf[r], push->world, push->rows, D, step & 1u, push->rank);
#pragma unroll
        for (int j = 0; j < J; ++j) {
          unsigned long long* at = part + grow * D + 16 * j + 4 * c;
          store_marked2(at, acc[j][0] * inv, acc[j][1] * inv, step + 1u);
          store_marked2(at + 2, acc[j][2] * inv, acc[j][3] * inv, step + 1u);
        }
        if (c == 0) store_marked(part + (int64_t)push->rows * D + grow, lse_out, step + 1u);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------
template <int KV, int D, int HB, bool SCALED, int NG, int WPC>
__global__ void __launch_bounds__(WPC * (HB + 1) * 32, 1)
stream_decode_kernel(const __grid_constant__ StreamParams sp, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v) {
  using C = StreamCfg<KV, D, HB, SCALED>;
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int kThreads = WPC * (HB + 1) * 32;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzled boxes need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw_addr);
  int* prefix = reinterpret_cast<int*>(smem + sp.prefix_off);
  unsigned short* nonempty = reinterpret_cast<unsigned short*>(smem + sp.count_off);  // [v]: sequences before v that have tiles
  int* bound = reinterpret_cast<int*>(smem + sp.bound_off);                            // the cells' boundaries
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + sp.misc_off);

  const Params& p = sp.p;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wl = warp / C::WARPS_PER_WORKER;    // worker within the CTA
  const int role = warp % C::WARPS_PER_WORKER;  // < HB: consumer of that head; == HB: producer
  const int nstage = sp.nstage;
  const uint32_t stage0 = base + (uint32_t)wl * nstage * C::STAGE_BYTES;
  const uint32_t full0 = base + sp.bar_off + (uint32_t)wl * nstage * 16;
  const uint32_t empty0 = full0 + nstage * 8;
  volatile int* meta = reinterpret_cast<volatile int*>(smem + sp.meta_off) + wl * nstage;

  // ---- tiles per virtual sequence, then an inclusive scan: prefix[v] = first tile of v ------
  const int nv = sp.nvseq;
  for (int v = tid; v < nv; v += kThreads) {
    const VseqInfo i = vseq_info(sp, v);
    prefix[v + 1] = i.hi > i.lo ? (i.hi - i.lo + kTileTokens - 1) / kTileTokens : 0;
  }
  // a cross-rank merge launched as a programmatic dependent may start now (a no-op otherwise)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // the producer's first copies wait for the two tensor-map descriptors: fetch them now, while the
  // CTA derives its share of the work
  if (role == HB && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&tm_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&tm_v) : "memory");
  }
  const bool pushing = sp.push.world > 0;
  volatile uint32_t* push_step = reinterpret_cast<volatile uint32_t*>(abort_flag + 2);
  if (tid == 0) {
    prefix[0] = 0;
    nonempty[0] = 0;
    *abort_flag = 0;
    // step counter of this rank's exchange buffer: its parity names the slots of this step
    *push_step = pushing ? *reinterpret_cast<volatile uint32_t*>(sp.push.peers.buf[sp.push.rank]) : 0u;
  }
  if (role == HB && lane == 0) {
    for (int s = 0; s < nstage; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, HB);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  volatile int* longest = abort_flag + 1;  // most tiles any virtual sequence has
  if (warp == 0) {
    int carry = 0, most = 0, ncarry = 0;
    for (int first = 1; first <= nv; first += 32) {
      const int idx = first + lane;
      int x = idx <= nv ? prefix[idx] : 0;
      int c = x > 0 ? 1 : 0;  // virtual sequences with tiles, counted alongside
      most = max(most, x);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(kFull, x, o);
        const int z = __shfl_up_sync(kFull, c, o);
        if (lane >= o) {
          x += y;
          c += z;
        }
      }
      if (idx <= nv) {
        prefix[idx] = x + carry;
        nonempty[idx] = (unsigned short)(c + ncarry);
      }
      carry += __shfl_sync(kFull, x, 31);
      ncarry += __shfl_sync(kFull, c, 31);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) most = max(most, __shfl_xor_sync(kFull, most, o));
    if (lane == 0) *longest = most;
  }
  __syncthreads();

  const int total = prefix[nv];
  const int workers = gridDim.x * WPC;
  const int w = blockIdx.x * WPC + wl;  // global worker id
  // Shares of equal COST, not of equal tile counts.  The end of a segment - partial result,
  // fence, ticket, perhaps a merge, the next request's query rows - costs a worker the time of
  // seg_cost tiles during which it consumes nothing, and a worker whose share crosses many short
  // requests pays it many times (per-CTA timelines of the ragged batch: 8 us at the median,
  // 18 us at the worst, and the launch ends with the worst).  So every virtual sequence with
  // tiles is charged its tiles plus seg_cost, the cost line is cut into equal parts, and each
  // boundary is carried back to the tile line: into the sequence the cut falls in, or to its
  // end when the cut falls into the surcharge.  A cut advances by more than seg_cost + 1, so no
  // cell between two others is empty.  Everything is a function of the lengths: all CTAs
  // derive the same boundaries, and two launches over the same lengths the same ones.
  // A small batch of short requests (fewer virtual sequences than workers, none longer than
  // kWholeTiles tiles) is dealt out whole, one request per worker, spread over the CTAs first:
  // every output row is then written directly, with no partial, ticket or merge on the way, and
  // nobody needs the boundaries (a call this short feels the barrier they would cost).
  const bool dealt_whole = sp.splits == 1 && nv <= workers && *longest <= kWholeTiles && !pushing;
  const int sc = sp.seg_cost;
  const long long total_c = (long long)total + (long long)sc * nonempty[nv];
  long long per_c = (total_c + workers - 1) / workers;
  if (per_c < kMinTilesPerWorker + sc) per_c = kMinTilesPerWorker + sc;
  for (int i = tid; i <= workers && !dealt_whole; i += kThreads) {
    const long long c = (long long)i * per_c;
    int tile = total;
    if (c < total_c) {
      int lo = 0, hi = nv;  // the last v whose cost prefix, prefix[v] + sc * nonempty[v], is <= c
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long)prefix[mid] + (long long)sc * nonempty[mid] <= c) lo = mid;
        else hi = mid;
      }
      const int off = (int)(c - ((long long)prefix[lo] + (long long)sc * nonempty[lo]));
      const int len = prefix[lo + 1] - prefix[lo];
      tile = prefix[lo] + (off < len ? off : len);
    }
    bound[i] = tile;
  }
  if (!dealt_whole) __syncthreads();  // the same for the whole CTA: it is derived from shared values
  CellMap cm;
  cm.bound = bound;
  cm.workers = workers;
  int g0, g1;
  if (dealt_whole) {
    const int mine = wl * gridDim.x + blockIdx.x;
    g0 = mine < nv ? prefix[mine] : total;
    g1 = mine < nv ? prefix[mine + 1] : total;
  } else {
    g0 = bound[w];
    g1 = bound[w + 1];
  }
  if (blockIdx.x == 0) {
    // requests without a single token are nobody's work: their rows are zero, their lse -inf
    for (int u = tid; u < sp.nhb * p.batch; u += kThreads) {
      if (prefix[(u + 1) * sp.splits] != prefix[u * sp.splits]) continue;
      const int b = u % p.batch, hb = u / p.batch;
      for (int h = hb * HB * p.group; h < (hb + 1) * HB * p.group; ++h) {
        for (int d = 0; d < D; ++d) {
          if (p.out) ((uint16_t*)p.out)[(int64_t)b * p.o_sb + (int64_t)h * p.o_sh + d] = 0;  // +0 in f16 and bf16
          if (p.res_o) p.res_o[((int64_t)b * p.hq + h) * D + d] = 0.f;
        }
        if (p.res_o) p.res_lse[(int64_t)b * p.hq + h] = -INFINITY;
      }
      if (pushing) {
        const uint32_t step = *push_step;
        for (int r = 0; r < sp.push.world; ++r) {
          unsigned long long* part = exchange_part(sp.push.peers.buf[r], sp.push.world, sp.push.rows, D, step & 1u,
                                                   sp.push.rank);
          for (int h = hb * HB * p.group; h < (hb + 1) * HB * p.group; ++h) {
            for (int d = 0; d < D; d += 2) store_marked2(part + ((int64_t)b * p.hq + h) * D + d, 0.f, 0.f, step + 1u);
            store_marked(part + (int64_t)sp.push.rows * D + (int64_t)b * p.hq + h, -INFINITY, step + 1u);
          }
        }
      }
    }
  }
  if (g0 >= g1) return;  // nothing for this worker (no barrier is used after this point)

  // =============================== producer warp =============================================
  if (role == HB) {
    constexpr uint32_t kTileTx = 2u * C::TILE_BYTES;
    int it = 0;
    int vbase = find_vseq(prefix, nv, g0);
    bool aborted = false;
    for (int g = g0; g < g1 && !aborted; g += 32) {
      const int myg = g + lane;
      const bool act = myg < g1;
      int mv = vbase;
      if (act)
        while (prefix[mv + 1] <= myg) ++mv;
      vbase = __shfl_sync(kFull, mv, 0);
      int phys = 0, tok = 0, hbi = 0, bad = 0;
      if (act) {
        const VseqInfo i = vseq_info(sp, mv);
        const int t0 = i.lo + (myg - prefix[mv]) * kTileTokens;
        const int pg = t0 / p.page;
        tok = t0 - pg * p.page;
        hbi = i.hb;
        phys = __ldg(p.block_table + (int64_t)i.b * p.bt_stride + pg);
        if ((unsigned)phys >= (unsigned)p.num_blocks) {
          if (p.status) atomicOr(p.status, PD_DEV_BAD_BLOCK);
          bad = 1;
          phys = 0;
        }
      }
      const int n = g1 - g < 32 ? g1 - g : 32;
      for (int i = 0; i < n; ++i, ++it) {
        const int st = it % nstage;
        const uint32_t ph = (uint32_t)(it / nstage) & 1u;
        const int phys_i = __shfl_sync(kFull, phys, i);
        const int tok_i = __shfl_sync(kFull, tok, i);
        const int hb_i = __shfl_sync(kFull, hbi, i);
        const int bad_i = __shfl_sync(kFull, bad, i);
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(empty0 + 8 * st, ph ^ 1u, p.status, abort_flag) ? 1 : 0;
          if (ok) {
            const uint32_t fb = full0 + 8 * st;
            const uint32_t dst = stage0 + (uint32_t)st * C::STAGE_BYTES;
            meta[st] = bad_i;
            if (bad_i) {
              mbar_arrive(fb);  // consumers skip the tile
            } else {
              mbar_arrive_expect_tx(fb, kTileTx + (SCALED ? 2u * sp.scale_tx_bytes : 0u));
#pragma unroll
              for (int c = 0; c < C::NC; ++c) {
                tma_load_4d(dst + c * C::CHUNK_BYTES, &tm_k, fb, c * C::BOX_ELEMS, tok_i,
                            hb_i * HB, phys_i);
                tma_load_4d(dst + C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_v, fb,
                            c * C::BOX_ELEMS, tok_i, hb_i * HB, phys_i);
              }
              if constexpr (SCALED) {
                const int64_t so = (int64_t)phys_i * p.sc_sb + (int64_t)tok_i * p.sc_st;
                bulk_load(dst + 2 * C::TILE_BYTES, p.k_scale + so, sp.scale_tx_bytes, fb);
                bulk_load(dst + 2 * C::TILE_BYTES + 1024, p.v_scale + so, sp.scale_tx_bytes, fb);
              }
            }
          }
        }
        if (!__shfl_sync(kFull, ok, 0)) {
          aborted = true;
          break;
        }
      }
    }
    if (lane == 0 && (aborted || *abort_flag)) {
      // give the copies still in flight a bounded chance to land before the CTA exits
      for (int k = 1; k <= nstage && k <= it; ++k) {
        const int ii = it - k;
        mbar_wait_slow(full0 + 8 * (ii % nstage), (uint32_t)(ii / nstage) & 1u, nullptr,
                       abort_flag, false);
      }
    }
    return;
  }

  // =============================== consumer warps ============================================
  const int gq = lane >> 2, tq = lane & 3;  // mma fragment coordinates
  const int hg = HB * p.group;              // query heads of one head block
  int it = 0;
  int v = find_vseq(prefix, nv, g0);
  int g = g0;
  bool aborted = false;

  while (g < g1 && !aborted) {
    while (prefix[v + 1] <= g) ++v;
    const VseqInfo vi = vseq_info(sp, v);
    const int vend = prefix[v + 1];
    const int seg_end = g1 < vend ? g1 : vend;
    int j = g - prefix[v];
    const bool whole = (j == 0) && (seg_end == vend) && (sp.splits == 1) && !pushing;
    const int kvh = vi.hb * HB + role;

    // ---- query rows of this kv head's group as B fragments: thread (g, t) holds head g (+8 per
    // n-tile), head_dim pairs of its k slots; heads >= group are zero --------------------------
    uint32_t qb[C::KSTEPS][NG][2];
    // Where the group's rows are one dense run, the warp first copies them into its own piece of
    // shared memory with 16-byte loads (a few full lines instead of sixteen 4-byte loads per lane
    // that each touch eight rows: what makes reading q from pinned host memory affordable, one
    // 128-byte read across the bus per line) and takes the fragments from there.
    constexpr uint32_t kQPitch = D * 2 + 16;
    const uint32_t qstage = sp.qstage_warp_bytes
                                ? base + sp.qstage_off + (uint32_t)(wl * HB + role) * sp.qstage_warp_bytes
                                : 0u;
    if (qstage) {
      constexpr int kRowChunks = D * 2 / 16;
      const uint4* src = reinterpret_cast<const uint4*>((const __half*)p.q + (int64_t)vi.b * p.q_sb +
                                                        (int64_t)kvh * p.group * p.q_sh);
      __syncwarp();  // the fragment reads of the segment before are over
      for (int i = lane; i < p.group * kRowChunks; i += 32)
        sts128(qstage + (uint32_t)(i / kRowChunks) * kQPitch + (uint32_t)(i % kRowChunks) * 16u, __ldg(src + i));
      __syncwarp();
    }
    // the two fetches are kept in two separate unrolled loops: one branch, not one per fragment
    auto fill_fragments = [&](auto&& fetch) {
#pragma unroll
      for (int ng = 0; ng < NG; ++ng) {
        const int head = 8 * ng + gq;
        const bool live = head < p.group;
#pragma unroll
        for (int ks = 0; ks < C::KSTEPS; ++ks) {
          int c_lo, c_hi;  // head_dim index of k slots (2t, 2t+1) and (2t+8, 2t+9)
          if constexpr (is_16bit(KV)) {
            c_lo = 16 * ks + 2 * tq;
            c_hi = c_lo + 8;
          } else {
            // every piece of an 8-bit row is read as its 16-byte chunks CPT*t .. CPT*t + CPT-1
            // (CPT = 2 for 128-byte pieces, 1 for 64-byte rows); k-step ks uses word ks % 4 of the
            // (ks / 4)-th chunk the thread reads, whose four elements fill its four k slots
            constexpr int CPT = C::CPR / 4;
            const int cj = ks >> 2;
            c_lo = C::PITCH * (cj / CPT) + 16 * (CPT * tq + cj % CPT) + 4 * (ks & 3);
            c_hi = c_lo + 2;
          }
          qb[ks][ng][0] = live ? fetch(head, c_lo) : 0u;
          qb[ks][ng][1] = live ? fetch(head, c_hi) : 0u;
        }
      }
    };
    if (qstage) {
      fill_fragments([&](int head, int col) { return lds32(qstage + (uint32_t)head * kQPitch + 2u * (uint32_t)col); });
    } else {
      const __half* qrows = (const __half*)p.q + (int64_t)vi.b * p.q_sb + (int64_t)kvh * p.group * p.q_sh;
      fill_fragments([&](int head, int col) {
        return __ldg(reinterpret_cast<const uint32_t*>(qrows + (int64_t)head * p.q_sh + col));
      });
    }
    // int8 keys meet the query on the integer tensor-core path.  Each query row is written as
    // step * (128 * hi + lo) with int8 digits hi in [-127, 127] and lo in [-64, 63], step =
    // max|q| / 16256: 15 bits relative to the row's largest element, finer than the fp16 inputs'
    // own spacing for all but their smallest elements.  The four elements of k-step ks are
    // packed as the bytes of qb[ks][.][0] (hi) and qb[ks][.][1] (lo); the scores of heads 2t and
    // 2t+1 are multiplied by those heads' steps afterwards.
    float qstep[NG][2];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
      qstep[ng][0] = qstep[ng][1] = 0.f;
      if constexpr (KV == PD_KV_I8) {
        float amax = 0.f;
#pragma unroll
        for (int ks = 0; ks < C::KSTEPS; ++ks) {
          const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&qb[ks][ng][0]));
          const float2 y = __half22float2(*reinterpret_cast<const __half2*>(&qb[ks][ng][1]));
          amax = fmaxf(fmaxf(amax, fmaxf(fabsf(x.x), fabsf(x.y))), fmaxf(fabsf(y.x), fabsf(y.y)));
        }
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));  // over head_dim of head g
        const float inv = amax > 0.f ? 16256.f / amax : 0.f;
        const float step = amax * (1.f / 16256.f);
#pragma unroll
        for (int ks = 0; ks < C::KSTEPS; ++ks) {
          const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&qb[ks][ng][0]));
          const float2 y = __half22float2(*reinterpret_cast<const __half2*>(&qb[ks][ng][1]));
          const float e[4] = {x.x, x.y, y.x, y.y};
          uint32_t hi_w = 0, lo_w = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int v = __float2int_rn(e[k] * inv);
            const int hi = (v + 64) >> 7;
            const int lo = v - (hi << 7);
            hi_w |= (uint32_t)(hi & 0xff) << (8 * k);
            lo_w |= (uint32_t)(lo & 0xff) << (8 * k);
          }
          qb[ks][ng][0] = hi_w;
          qb[ks][ng][1] = lo_w;
        }
        qstep[ng][0] = __shfl_sync(kFull, step, 4 * (2 * tq));
        qstep[ng][1] = __shfl_sync(kFull, step, 4 * (2 * tq + 1));
      }
    }

    // The query rows of this worker's NEXT segment, into L1 now: their load at that segment's
    // start is otherwise a round trip to HBM during which the warp consumes nothing (the KV
    // stream has long pushed q out of L2).  One 128-byte line per lane.
    if (seg_end < g1 && v + 1 < nv) {
      const VseqInfo nx = vseq_info(sp, v + 1);
      const int lines = (p.group * D * 2 + 127) / 128;
      if (lane < lines) {
        const char* nq = (const char*)p.q + 2 * ((int64_t)nx.b * p.q_sb +
                                                 (int64_t)(nx.hb * HB + role) * p.group * p.q_sh);
        asm volatile("prefetch.global.L1 [%0];" ::"l"(nq + 128 * lane));
      }
    }

    float m[NG][2], l[NG][2];
    float o[C::MT][NG][4];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
      m[ng][0] = m[ng][1] = -INFINITY;
      l[ng][0] = l[ng][1] = 0.f;
    }
#pragma unroll
    for (int mt = 0; mt < C::MT; ++mt)
#pragma unroll
      for (int ng = 0; ng < NG; ++ng) o[mt][ng][0] = o[mt][ng][1] = o[mt][ng][2] = o[mt][ng][3] = 0.f;
    float psum[NG][4];  // int8 pages: running column sums of P^T (see consume_tile)
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) psum[ng][0] = psum[ng][1] = psum[ng][2] = psum[ng][3] = 0.f;

    // 8-bit tiles with a deep ring (five stages or more) are taken two at a time: one softmax
    // step per 32 tokens and two independent score chains per warp.  With fewer stages the
    // second stage held by the consumers would cost the producer its lead.  16-bit rows of up to
    // 128 bytes (head_dim 64 and below: small stages, a deep ring) do the same: their requests
    // are short and a warp's chain of softmax steps is most of such a call.
    constexpr bool kPairs = !is_16bit(KV) || D <= 64;
    const bool pairs = kPairs && nstage >= 5;
    while (g < seg_end) {
      const int st = it % nstage;
      if (!mbar_wait(full0 + 8 * st, (uint32_t)(it / nstage) & 1u, p.status, abort_flag)) {
        aborted = true;
        break;
      }
      const uint32_t sbase = stage0 + (uint32_t)st * C::STAGE_BYTES;
      const int remaining = vi.hi - (vi.lo + j * kTileTokens);
      if constexpr (kPairs) {
        if (pairs && g + 1 < seg_end) {
          const int st1 = (it + 1) % nstage;
          if (!mbar_wait(full0 + 8 * st1, (uint32_t)((it + 1) / nstage) & 1u, p.status, abort_flag)) {
            aborted = true;
            break;
          }
          if (meta[st] == 0 && meta[st1] == 0) {
            const uint32_t sbase1 = stage0 + (uint32_t)st1 * C::STAGE_BYTES;
            const uint32_t kb[2] = {sbase + role * (kTileTokens * C::PITCH),
                                    sbase1 + role * (kTileTokens * C::PITCH)};
            const uint32_t sc[2] = {sbase + 2 * C::TILE_BYTES + kvh * 2, sbase1 + 2 * C::TILE_BYTES + kvh * 2};
            const int remaining1 = remaining - kTileTokens;  // >= 1: the next tile is of this request
            if (remaining1 >= kTileTokens)
              consume_tile<KV, D, HB, SCALED, NG, false, 2>(kb, sc, p.hkv, kTileTokens, p.scale_log2,
                                                            lane, qb, qstep, m, l, o, psum);
            else
              consume_tile<KV, D, HB, SCALED, NG, true, 2>(kb, sc, p.hkv, remaining1, p.scale_log2,
                                                           lane, qb, qstep, m, l, o, psum);
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(empty0 + 8 * st);
              mbar_arrive(empty0 + 8 * st1);
            }
            g += 2;
            j += 2;
            it += 2;
            continue;
          }
          // a tile with a bad block id: take the two one by one (the second wait returns at once)
        }
      }
      if (meta[st] == 0) {
        const uint32_t kb[1] = {sbase + role * (kTileTokens * C::PITCH)};
        const uint32_t sc[1] = {sbase + 2 * C::TILE_BYTES + kvh * 2};
        if (remaining >= kTileTokens)
          consume_tile<KV, D, HB, SCALED, NG, false>(kb, sc, p.hkv, kTileTokens, p.scale_log2,
                                                     lane, qb, qstep, m, l, o, psum);
        else
          consume_tile<KV, D, HB, SCALED, NG, true>(kb, sc, p.hkv, remaining, p.scale_log2,
                                                    lane, qb, qstep, m, l, o, psum);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * st);
      ++g;
      ++j;
      ++it;
    }
    if (aborted) break;

    // ---- segment epilogue: the thread owns heads 2t, 2t+1 (+8 per n-tile) -----------------------
    if constexpr (KV == PD_KV_I8) {
      // the surplus of the biased int8 values: 1152 times the column sums of P^T, rows alike
#pragma unroll
      for (int mt = 0; mt < C::MT; ++mt) {
#pragma unroll
        for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
          for (int r = 0; r < 4; ++r) o[mt][ng][r] = fmaf(-1152.f, psum[ng][r], o[mt][ng][r]);
        }
      }
    }
    const float unscale = SCALED ? (1.f / 256.f) : 1.f;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float lsum = l[ng][e];
#pragma unroll
        for (int sh = 4; sh < 32; sh <<= 1) lsum += __shfl_xor_sync(kFull, lsum, sh);
        const int head = 8 * ng + 2 * tq + e;
        if (head >= p.group) continue;
        const float inv = lsum > 0.f ? unscale / lsum : 0.f;
        const float lse = lsum > 0.f ? m[ng][e] + log2f(lsum) : -INFINITY;
        const int hq = kvh * p.group + head;
        __half* dst16 = nullptr;
        float* dst32 = nullptr;
        if (whole) {
          if (p.out) dst16 = (__half*)p.out + (int64_t)vi.b * p.o_sb + (int64_t)hq * p.o_sh;
          if (p.res_o) {
            dst32 = p.res_o + ((int64_t)vi.b * p.hq + hq) * D;
            if (gq == 0) p.res_lse[(int64_t)vi.b * p.hq + hq] = lse;
          }
        } else {
          const int64_t slot_row = (int64_t)(w + v) * hg + role * p.group + head;
          dst32 = p.part_o + slot_row * D;
          if (gq == 0) p.part_lse[slot_row] = lse;
        }
        if constexpr (is_16bit(KV)) {
          // m-tile mt holds head_dim 16*mt + g (regs 0, 1) and 16*mt + g + 8 (regs 2, 3)
#pragma unroll
          for (int mt = 0; mt < C::MT; ++mt) {
            const float x = o[mt][ng][e] * inv, y = o[mt][ng][2 + e] * inv;
            const int col = 16 * mt + gq;
            if (dst16) {
              store_io<KV>(dst16, col, x);
              store_io<KV>(dst16, col + 8, y);
            }
            if (dst32) {
              dst32[col] = x;
              dst32[col + 8] = y;
            }
          }
        } else {
          // the thread's BPT = PITCH / 8 contiguous columns of every piece, eight at a time:
          // word i of piece c came from m-tiles c*(PITCH/16) + 2*i and + 1 (rows g and g + 8)
          constexpr int WPT = C::PITCH / 32;
#pragma unroll
          for (int c = 0; c < C::NC; ++c) {
#pragma unroll
            for (int i = 0; i < WPT; i += 2) {
              float x[8];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int mt = c * (C::PITCH / 16) + 2 * i + k;
                x[2 * k] = o[mt][ng][e] * inv;
                x[2 * k + 1] = o[mt][ng][2 + e] * inv;
              }
              const int col = c * C::PITCH + (C::PITCH / 8) * gq + 4 * i;
              if (dst16) {
                uint4 pk;
                pk.x = pack_io2<KV>(x[0], x[1]);
                pk.y = pack_io2<KV>(x[2], x[3]);
                pk.z = pack_io2<KV>(x[4], x[5]);
                pk.w = pack_io2<KV>(x[6], x[7]);
                *reinterpret_cast<uint4*>(dst16 + col) = pk;
              }
              if (dst32) {
                *reinterpret_cast<float4*>(dst32 + col) = make_float4(x[0], x[1], x[2], x[3]);
                *reinterpret_cast<float4*>(dst32 + col + 4) = make_float4(x[4], x[5], x[6], x[7]);
              }
            }
          }
        }
      }
    }
    if (!whole) {
      // Ticket: every segment of this (request, kv head) adds one after its partial is visible;
      // whoever completes the count merges them all.  Nobody waits for anybody.
      __threadfence();
      __syncwarp();
      const int v0 = (vi.hb * p.batch + vi.b) * sp.splits;
      int* unit_ticket = sp.tickets + (int64_t)vi.b * p.hkv + kvh;
      // An unsplit request cut over more than kMergeRadix workers (one long request can span
      // every worker) is merged in two levels: chunks of kMergeRadix consecutive segments
      // first, each by the warp that completes the chunk, into the chunk's first slot; then
      // the chunk results by the warp that completes the unit.  The chunk merges of one
      // request run on different SMs at the same time.
      int wfirst = 0, nseg = 0;
      if (sp.splits == 1) {
        wfirst = cm.of(prefix[v0]);
        nseg = cm.of(prefix[v0 + 1] - 1) - wfirst + 1;
      }
      if (nseg > kMergeRadix) {
        const int chunk = (w - wfirst) / kMergeRadix;
        const int csize = min(kMergeRadix, nseg - chunk * kMergeRadix);
        const int nchunk = (nseg + kMergeRadix - 1) / kMergeRadix;
        const int cslot = wfirst + chunk * kMergeRadix + v0;
        int done = 0;
        if (lane == 0) {
          int* chunk_ticket = sp.tickets + (int64_t)p.batch * p.hkv + (int64_t)cslot * HB + role;
          done = atomicAdd(chunk_ticket, 1) + 1 == csize;
          if (done) *chunk_ticket = 0;
        }
        if (__shfl_sync(kFull, done, 0)) {
          __threadfence();
          merge_unit<KV, D>(p, prefix, cm, v0, 1, hg, role, vi.b, kvh, lane, cslot, csize, 1, cslot);
          __threadfence();
          __syncwarp();
          int last = 0;
          if (lane == 0) {
            last = atomicAdd(unit_ticket, 1) + 1 == nchunk;
            if (last) *unit_ticket = 0;
          }
          if (__shfl_sync(kFull, last, 0)) {
            __threadfence();
            merge_unit<KV, D>(p, prefix, cm, v0, 1, hg, role, vi.b, kvh, lane, wfirst + v0, nchunk,
                              kMergeRadix, -1, pushing ? &sp.push : nullptr, *push_step);
          }
        }
      } else {
        int last = 0;
        if (lane == 0) {
          int expected = 0;
          for_each_segment(prefix, cm, v0, sp.splits, [&](int) { ++expected; });
          last = atomicAdd(unit_ticket, 1) + 1 == expected;
          if (last) *unit_ticket = 0;  // leave the counter as it was found
        }
        if (__shfl_sync(kFull, last, 0)) {
          __threadfence();
          merge_unit<KV, D>(p, prefix, cm, v0, sp.splits, hg, role, vi.b, kvh, lane, 0, 0, 1, -1,
                            pushing ? &sp.push : nullptr, *push_step);
        }
      }
    }
    ++v;
  }
}

}  // namespace pd
