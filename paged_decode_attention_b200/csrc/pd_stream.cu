// Host side of the streaming decode kernel (pd_stream_kernel.cuh): which requests it serves, its
// shared-memory and scratch plans, TMA tensor maps, kernel dispatch, the allocation-free entry
// point pd_decode_static and the bounded-wait self-test.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "pd_stream.h"
#include "pd_stream_kernel.cuh"

namespace pd {

// One translation unit per page element type holds that type's kernel instantiations.
#define PD_STREAM_LAUNCHER(name)                                                              \
  cudaError_t name(int head_dim, int hb, const StreamParams& sp, const CUtensorMap& mk,      \
                   const CUtensorMap& mv, int grid, uint32_t smem, cudaStream_t st)
PD_STREAM_LAUNCHER(stream_launch_f16);
PD_STREAM_LAUNCHER(stream_launch_bf16);
PD_STREAM_LAUNCHER(stream_launch_e5m2);
PD_STREAM_LAUNCHER(stream_launch_e5m2_scaled);
PD_STREAM_LAUNCHER(stream_launch_i8);
#undef PD_STREAM_LAUNCHER

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static uint64_t round_up64(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

static int head_block(int hkv) {
  for (int hb = 8; hb > 1; hb >>= 1)
    if (hkv % hb == 0) return hb;
  return 1;
}

struct Shape {
  int hb, nhb, wpc, splits, nvseq, stage_bytes, seg_cost;
  uint32_t qwarp_bytes;  // query staging one consumer warp would need; 0: the group's rows are not one dense run
  bool scaled;
};

// Workers (CTAs x workers per CTA) the cells' boundary table in shared memory is sized for.
constexpr int kMaxWorkers = 1024;

static Shape derive(const PdDecodeArgs* a) {
  Shape s;
  s.hb = head_block(a->num_kv_heads);
  // head_dim 256: a consumer thread holds 64 accumulator and 32 query registers per n-tile, and
  // at 16 bits a stage of 8 consumer warps' worth would be 128 KB; so at most four heads per
  // block and four consumer warps per CTA
  const bool wide = a->head_dim == 256;
  if (wide && s.hb > 4) s.hb = 4;
  s.nhb = a->num_kv_heads / s.hb;
  s.wpc = wide ? 4 / s.hb : base_workers_per_cta(s.hb);
  s.splits = a->num_splits > 0 ? a->num_splits : 1;
  const long long nv = (long long)s.nhb * a->batch * s.splits;
  s.nvseq = nv > INT32_MAX ? INT32_MAX : (int)nv;
  s.scaled = a->k_scale != nullptr;
  const int eb = is_16bit(a->kv_dtype) ? 2 : 1;
  // a tile of K (or V) is hb heads x 16 tokens x the row, whatever pieces the row is moved in
  s.stage_bytes = 2 * s.hb * kTileTokens * a->head_dim * eb + (s.scaled ? 2048 : 0);
  // What one segment end costs a worker, in tiles' worth of its time: the shares of the tile line
  // are balanced with it.  Per-CTA timelines put an end at 3-4 us and a tile at 1.5 us (16-bit
  // pages) or 0.8 us (8-bit pages) of a worker's time, i.e. 2 and 5 tiles; swept on the full-size
  // batches (0, 2, 4, 8, 12), the launches were shortest at 8 (ragged fp16: -1.2 %; uniform fp16:
  // -0.6 % from 4 upwards) and at 12 (int8: -1.0 %) - an end also delays the worker's producer.
  s.seg_cost = (a->flags & PD_FLAG_EQUAL_TILE_SHARES) ? 0 : (eb == 2 ? 8 : 12);
  // on request (PD_FLAG_STAGE_Q) the kernel stages a group's query rows with 16-byte loads, when
  // they are one aligned dense run
  const bool q_dense = (a->flags & PD_FLAG_STAGE_Q) && a->q_stride_h == a->head_dim && ((uintptr_t)a->q % 16) == 0 &&
                       (a->q_stride_b * 2) % 16 == 0;
  s.qwarp_bytes = q_dense ? (uint32_t)(a->num_q_heads / a->num_kv_heads) * (uint32_t)(a->head_dim * 2 + 16) : 0u;
  return s;
}

struct SmemPlan {
  int nstage;
  uint32_t bar_off, meta_off, misc_off, prefix_off, count_off, bound_off, qstage_off, qstage_warp_bytes, total;
};

static bool plan_smem(const Shape& s, SmemPlan& sm) {
  const uint32_t fixed_per_stage = (uint32_t)s.wpc * (16 + 4);
  // lengths' prefix (int), count of non-empty sequences (u16), the cells' boundaries (int)
  const uint32_t tail = 64 + (uint32_t)(s.nvseq + 2) * 6 + 16 + (uint32_t)(kMaxWorkers + 2) * 4 +
                        1024 /* alignment slack */;
  int n = kMaxStages;
  for (; n >= 2; --n) {
    const uint64_t need = (uint64_t)n * s.wpc * s.stage_bytes + (uint64_t)n * fixed_per_stage + tail;
    if (need <= (uint64_t)kSmemLimit) break;
  }
  if (n < 2) return false;
  sm.nstage = n;
  sm.bar_off = (uint32_t)n * s.wpc * s.stage_bytes;
  sm.meta_off = sm.bar_off + (uint32_t)n * s.wpc * 16;
  sm.misc_off = (sm.meta_off + (uint32_t)n * s.wpc * 4 + 15u) & ~15u;
  sm.prefix_off = sm.misc_off + 16;
  sm.count_off = sm.prefix_off + (uint32_t)(s.nvseq + 2) * 4;
  sm.bound_off = (sm.count_off + (uint32_t)(s.nvseq + 2) * 2 + 15u) & ~15u;
  sm.total = sm.bound_off + (uint32_t)(kMaxWorkers + 2) * 4 + 1024;
  // query staging only where it costs no stage of the ring
  sm.qstage_off = (sm.bound_off + (uint32_t)(kMaxWorkers + 2) * 4 + 15u) & ~15u;
  sm.qstage_warp_bytes = 0;
  const uint32_t qbytes = (uint32_t)(s.wpc * s.hb) * s.qwarp_bytes;
  if (qbytes && (uint64_t)sm.qstage_off + qbytes + 1024 <= (uint64_t)kSmemLimit) {
    sm.qstage_warp_bytes = s.qwarp_bytes;
    sm.total = sm.qstage_off + qbytes + 1024;
  }
  return true;
}

int stream_supports(const PdDecodeArgs* a) {
  // bf16 pages go with bf16 q/out, every other page type with f16 q/out
  if ((a->kv_dtype == PD_KV_BF16) != (a->io_dtype == PD_IO_BF16)) return PD_ERR_UNSUPPORTED;
  const int eb = is_16bit(a->kv_dtype) ? 2 : 1;
  const int rowb = a->head_dim * eb;
  // rows of 64 bytes or of whole 128-byte pieces: head_dim 32..256 on 16-bit pages, 64..256
  // on 8-bit pages
  if (rowb != 64 && rowb != 128 && rowb != 256 && rowb != 512) return PD_ERR_UNSUPPORTED;
  if (a->head_dim > 256) return PD_ERR_UNSUPPORTED;
  if (a->batch <= 0) return PD_ERR_UNSUPPORTED;
  const int group = a->num_q_heads / a->num_kv_heads;
  if (group > 16) return PD_ERR_UNSUPPORTED;
  if (a->block_size % kTileTokens != 0 || a->block_size > 256) return PD_ERR_UNSUPPORTED;
  const int block_n = a->block_n ? a->block_n : 64;
  if (block_n % kTileTokens != 0) return PD_ERR_UNSUPPORTED;
  // 32-bit fragment loads of q, vector stores of out
  if (((uintptr_t)a->q % 4) || a->q_stride_b % 2 || a->q_stride_h % 2) return PD_ERR_UNSUPPORTED;
  if (a->out && (((uintptr_t)a->out % 16) || a->out_stride_b % 8 || a->out_stride_h % 8))
    return PD_ERR_UNSUPPORTED;
  if (a->result_f32 && (((uintptr_t)a->result_f32 % 16) || ((uintptr_t)a->result_lse % 4)))
    return PD_ERR_UNSUPPORTED;
  if (a->k_scale) {
    if (a->scale_stride_token != a->num_kv_heads || (a->scale_stride_block * 2) % 16 ||
        ((uintptr_t)a->k_scale % 16) || ((uintptr_t)a->v_scale % 16) || a->num_kv_heads > 32)
      return PD_ERR_UNSUPPORTED;
  }
  const Shape s = derive(a);
  if ((long long)s.nhb * a->batch * s.splits > kMaxVseq) return PD_ERR_UNSUPPORTED;
  SmemPlan sm;
  if (!plan_smem(s, sm)) return PD_ERR_UNSUPPORTED;
  // tensor-map limits: 16-byte aligned base and strides, strides below 2^40 bytes
  if (((uintptr_t)a->k_cache % 16) || ((uintptr_t)a->v_cache % 16) || (a->kv_stride_block * eb) % 16 ||
      (a->kv_stride_token * eb) % 16 || (a->kv_stride_head * eb) % 16)
    return PD_ERR_UNSUPPORTED;
  if ((uint64_t)a->kv_stride_block * eb >= (1ull << 40) || (uint64_t)a->kv_stride_token * eb >= (1ull << 40) ||
      (uint64_t)a->kv_stride_head * eb >= (1ull << 40))
    return PD_ERR_UNSUPPORTED;
  return PD_OK;
}

struct WorkspaceLayout {
  uint64_t ticket_off, ticket_bytes, lse_off, o_off, total;
  int slots;
};

static WorkspaceLayout workspace_layout(const PdDecodeArgs* a, const Shape& s, int sm_count) {
  WorkspaceLayout w;
  const int group = a->num_q_heads / a->num_kv_heads;
  w.slots = sm_count * s.wpc + s.nvseq;
  w.ticket_off = 0;
  // one counter per (request, kv head), then one per (slot, kv head of the block) for the
  // chunks of deep merges
  w.ticket_bytes = ((uint64_t)a->batch * a->num_kv_heads + (uint64_t)w.slots * s.hb) * 4;
  w.lse_off = round_up64(w.ticket_bytes, 256);
  w.o_off = w.lse_off + round_up64((uint64_t)w.slots * s.hb * group * 4, 256);
  w.total = w.o_off + round_up64((uint64_t)w.slots * s.hb * group * a->head_dim * 4, 256);
  return w;
}

uint64_t stream_workspace_bytes(const PdDecodeArgs* a, int sm_count) {
  return workspace_layout(a, derive(a), sm_count).total;
}

uint64_t stream_counter_bytes(const PdDecodeArgs* a, int sm_count) {
  return workspace_layout(a, derive(a), sm_count).ticket_bytes;
}

// ---- tensor maps --------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return (EncodeFn)ptr;
  }();
  return fn;
}

struct MapKey {
  const void* base;
  int64_t sb, st, sh;
  int32_t d, page, hkv, nb, hb, kv;
  bool operator==(const MapKey& o) const {
    return base == o.base && sb == o.sb && st == o.st && sh == o.sh && d == o.d && page == o.page &&
           hkv == o.hkv && nb == o.nb && hb == o.hb && kv == o.kv;
  }
};

// Tensor map over one cache tensor with dimensions ordered (head_dim, token, head, block) so
// that a box lands in shared memory as [head][token][128 bytes] (64 bytes when that is the
// whole row): a head's 16 token rows are consecutive rows and the swizzle of the row's width
// spreads them over all banks.  Encoded
// straight into caller storage; allocates nothing.
static bool encode_tensor_map_in_place(const MapKey& k, CUtensorMap* out) {
  EncodeFn enc = encode_fn();
  if (!enc) return false;
  const int eb = is_16bit(k.kv) ? 2 : 1;
  const cuuint64_t dims[4] = {(cuuint64_t)k.d, (cuuint64_t)k.page, (cuuint64_t)k.hkv, (cuuint64_t)k.nb};
  const cuuint64_t strides[3] = {(cuuint64_t)k.st * eb, (cuuint64_t)k.sh * eb, (cuuint64_t)k.sb * eb};
  const int pitch = k.d * eb < 128 ? k.d * eb : 128;
  const cuuint32_t box[4] = {(cuuint32_t)(pitch / eb), (cuuint32_t)kTileTokens, (cuuint32_t)k.hb, 1u};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(out, k.kv == PD_KV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : eb == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 4,
             const_cast<void*>(k.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             pitch == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same through a small cache keyed by everything the encoding depends on.
static bool get_tensor_map(const MapKey& k, CUtensorMap* out) {
  static std::mutex mu;
  static std::vector<std::pair<MapKey, CUtensorMap>> cache;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (auto& e : cache)
      if (e.first == k) {
        *out = e.second;
        return true;
      }
  }
  if (!encode_tensor_map_in_place(k, out)) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() >= 64) cache.erase(cache.begin());
  cache.emplace_back(k, *out);
  return true;
}

// Fills the kernel's parameter block for scratch at `scratch`, clears the arrival counters on the
// stream and launches the instantiation that serves the arguments.  Shared by pd_decode and
// pd_decode_static, which differ only in where the scratch lives and how the tensor maps are made.
static int launch_stream(const PdDecodeArgs* a, const Params& p, const Shape& s, const SmemPlan& sm,
                         const WorkspaceLayout& wl, char* scratch, const CUtensorMap& mk,
                         const CUtensorMap& mv, int sm_count, bool counters_zero = false,
                         const PushTargets* push = nullptr) {
  StreamParams sp;
  sp.p = p;
  sp.p.num_splits = s.splits;
  sp.p.part_lse = (float*)(scratch + wl.lse_off);
  sp.p.part_o = (float*)(scratch + wl.o_off);
  sp.nvseq = s.nvseq;
  sp.nhb = s.nhb;
  sp.splits = s.splits;
  sp.nstage = sm.nstage;
  sp.wpc = s.wpc;
  sp.bar_off = sm.bar_off;
  sp.meta_off = sm.meta_off;
  sp.misc_off = sm.misc_off;
  sp.prefix_off = sm.prefix_off;
  sp.count_off = sm.count_off;
  sp.bound_off = sm.bound_off;
  sp.qstage_off = sm.qstage_off;
  sp.qstage_warp_bytes = sm.qstage_warp_bytes;
  sp.seg_cost = s.seg_cost;
  sp.tickets = (int32_t*)(scratch + wl.ticket_off);
  sp.scale_tx_bytes = (uint32_t)(kTileTokens * a->num_kv_heads * 2);
  if (push) sp.push = *push;
  else memset(&sp.push, 0, sizeof(sp.push));

  const cudaStream_t st = (cudaStream_t)a->stream;
  // The arrival counters of the in-kernel merge start at zero.  Every kernel leaves them at
  // zero, so a caller that vouches for a workspace it cleared once skips the memset node.
  if (!counters_zero && cudaMemsetAsync(sp.tickets, 0, wl.ticket_bytes, st) != cudaSuccess) return PD_ERR_CUDA;
  cudaError_t e;
  switch (a->kv_dtype) {
    case PD_KV_F16: e = stream_launch_f16(a->head_dim, s.hb, sp, mk, mv, sm_count, sm.total, st); break;
    case PD_KV_BF16: e = stream_launch_bf16(a->head_dim, s.hb, sp, mk, mv, sm_count, sm.total, st); break;
    case PD_KV_E5M2:
      e = s.scaled ? stream_launch_e5m2_scaled(a->head_dim, s.hb, sp, mk, mv, sm_count, sm.total, st)
                   : stream_launch_e5m2(a->head_dim, s.hb, sp, mk, mv, sm_count, sm.total, st);
      break;
    default: e = stream_launch_i8(a->head_dim, s.hb, sp, mk, mv, sm_count, sm.total, st); break;
  }
  return e == cudaSuccess ? PD_OK : PD_ERR_CUDA;
}

static MapKey map_key(const PdDecodeArgs* a, const Shape& s, const void* base) {
  return MapKey{base, a->kv_stride_block, a->kv_stride_token, a->kv_stride_head, a->head_dim,
                a->block_size, a->num_kv_heads, a->num_blocks, s.hb, a->kv_dtype};
}

int stream_run(const PdDecodeArgs* a, Params& p, int sm_count, const PushTargets* push) {
  const Shape s = derive(a);
  SmemPlan sm;
  if (!plan_smem(s, sm)) return PD_ERR_UNSUPPORTED;
  if ((long long)sm_count * s.wpc > kMaxWorkers) return PD_ERR_UNSUPPORTED;
  const WorkspaceLayout wl = workspace_layout(a, s, sm_count);
  if (!a->workspace || a->workspace_bytes < wl.total) return PD_ERR_WORKSPACE;
  CUtensorMap mk, mv;
  if (!get_tensor_map(map_key(a, s, a->k_cache), &mk) || !get_tensor_map(map_key(a, s, a->v_cache), &mv))
    return PD_ERR_CUDA;
  return launch_stream(a, p, s, sm, wl, (char*)a->workspace, mk, mv, sm_count,
                       (a->flags & PD_FLAG_COUNTERS_ZERO) != 0, push);
}

// ---------------------------------------------------------------------------------------------
// pd_decode_static: the streaming decode with its scratch in library-owned device memory
// ---------------------------------------------------------------------------------------------
// Scratch of pd_decode_static.  It is part of the loaded module: every GPU that loads this
// library holds these bytes from load until the process exits.  All calls share it.
static __device__ __align__(256) unsigned char g_static_scratch[PD_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, looked up once per device.  In host
// code the array's name is only a handle for the runtime, not an address a kernel can use; the
// address has to come from cudaGetSymbolAddress with the target device current.
static void* static_scratch_address() {
  static std::mutex mu;
  static void* address[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!address[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    address[dev] = ptr;
  }
  return address[dev];
}

static int stream_run_static(const PdDecodeArgs* a, Params& p, int sm_count) {
  const Shape s = derive(a);
  SmemPlan sm;
  if (!plan_smem(s, sm)) return PD_ERR_UNSUPPORTED;
  if ((long long)sm_count * s.wpc > kMaxWorkers) return PD_ERR_UNSUPPORTED;
  const WorkspaceLayout wl = workspace_layout(a, s, sm_count);
  if (wl.total > (uint64_t)PD_STATIC_SCRATCH_BYTES) return PD_ERR_TOO_LARGE;
  char* scratch = (char*)static_scratch_address();
  if (!scratch) return PD_ERR_CUDA;
  // Only the arrival counters have to start at zero; launch_stream clears them on the stream
  // ahead of the kernel.  Every partial slot is written before the merge inside the kernel
  // reads it.  The tensor maps are encoded in place: no cache, so nothing is allocated.
  CUtensorMap mk, mv;
  if (!encode_tensor_map_in_place(map_key(a, s, a->k_cache), &mk) ||
      !encode_tensor_map_in_place(map_key(a, s, a->v_cache), &mv))
    return PD_ERR_CUDA;
  return launch_stream(a, p, s, sm, wl, scratch, mk, mv, sm_count);
}

// A wait nobody ends, on purpose: one warp initialises an mbarrier that no thread and no copy
// ever arrives on and waits for it with the kernel's own bounded wait.  The wait must give up
// after `limit_ns`, raise PD_DEV_TIMEOUT in the status word and return normally.
__global__ void bounded_wait_selftest_kernel(uint32_t* status, unsigned long long limit_ns) {
  __shared__ unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(addr, 1);
    fence_barrier_init();
  }
  __syncthreads();
  mbar_wait_slow(addr, 0, status, &abort_flag, true, limit_ns);
}

}  // namespace pd

extern "C" PD_API int pd_selftest_bounded_wait(uint32_t* status, uint64_t limit_ns, void* stream) {
  if (!status || limit_ns == 0 || limit_ns > 1000000000ull) return PD_ERR_INVALID_ARG;
  pd::bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? PD_OK : PD_ERR_CUDA;
}

// Decode step for callers that cannot hand over scratch memory: see include/paged_decode.h.
// The first call on a device looks up the scratch array's device address (one
// cudaGetSymbolAddress with that device current); make that first call outside any stream
// capture.  No cudaMalloc, cudaFree or other allocating routine is called, on any call.
extern "C" PD_API int pd_decode_static(const PdDecodeArgs* args) {
  using namespace pd;
  const int rc = validate(args);
  if (rc != PD_OK) return rc;
  const int why = stream_supports(args);
  if (why != PD_OK) return why;
  const int sms = resolve_sm_count(args);
  if (sms <= 0) return PD_ERR_CUDA;
  Params p;
  fill_params(args, p);
  return stream_run_static(args, p, sms);
}
