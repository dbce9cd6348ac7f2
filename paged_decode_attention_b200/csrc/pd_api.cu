// C ABI of the library (include/paged_decode.h): argument validation, kernel selection and
// launches.  Everything here runs on the host; no device memory is allocated.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "pd_common.cuh"
#include "pd_cache_write.cuh"
#include "pd_exchange.cuh"
#include "pd_merge.cuh"
#include "pd_simple.cuh"
#include "pd_stream.h"

namespace pd {

static int cached_sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

static bool aligned(const void* p, uintptr_t a) { return ((uintptr_t)p % a) == 0; }

// The address under which the current device reaches page-locked host memory at `host`, or
// nullptr when `host` is ordinary (pageable) memory or memory of another kind.
static void* device_view_of_host(const void* host) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

static int elem_bytes(int kv) { return (kv == PD_KV_F16 || kv == PD_KV_BF16) ? 2 : 1; }

// Checks everything that can be checked without touching the device.
int validate(const PdDecodeArgs* a, bool need_output) {
  if (!a) return PD_ERR_INVALID_ARG;
  if (!a->q || !a->k_cache || !a->v_cache || !a->block_table || !a->seq_lens)
    return PD_ERR_INVALID_ARG;
  if (need_output && !a->out && !a->result_f32) return PD_ERR_INVALID_ARG;
  if ((a->result_f32 == nullptr) != (a->result_lse == nullptr)) return PD_ERR_INVALID_ARG;
  if (a->batch < 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0 || a->head_dim <= 0)
    return PD_ERR_INVALID_ARG;
  if (a->num_q_heads % a->num_kv_heads != 0) return PD_ERR_INVALID_ARG;
  if (a->block_size <= 0 || a->num_blocks <= 0 || a->max_blocks_per_seq <= 0)
    return PD_ERR_INVALID_ARG;
  if (a->kv_dtype < PD_KV_F16 || a->kv_dtype > PD_KV_I8) return PD_ERR_INVALID_ARG;
  if (a->io_dtype != PD_IO_F16 && a->io_dtype != PD_IO_BF16) return PD_ERR_INVALID_ARG;
  if (a->kernel < PD_KERNEL_AUTO || a->kernel > PD_KERNEL_STREAM) return PD_ERR_INVALID_ARG;
  if (a->num_splits < 0 || a->num_splits > 1024) return PD_ERR_INVALID_ARG;
  const int block_n = a->block_n ? a->block_n : 64;
  if (block_n <= 0 || block_n % a->block_size != 0) return PD_ERR_INVALID_ARG;
  const bool has_scale = a->k_scale != nullptr;
  if ((a->k_scale == nullptr) != (a->v_scale == nullptr)) return PD_ERR_INVALID_ARG;
  if (a->kv_dtype == PD_KV_I8 && !has_scale) return PD_ERR_INVALID_ARG;
  if ((a->kv_dtype == PD_KV_F16 || a->kv_dtype == PD_KV_BF16) && has_scale)
    return PD_ERR_INVALID_ARG;
  if (a->block_table_stride < a->max_blocks_per_seq) return PD_ERR_INVALID_ARG;
  if (a->head_dim != 32 && a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256)
    return PD_ERR_UNSUPPORTED;
  // vector loads: rows and base pointers 16-byte aligned
  const int eb = elem_bytes(a->kv_dtype);
  if ((a->kv_stride_block * eb) % 16 || (a->kv_stride_token * eb) % 16 ||
      (a->kv_stride_head * eb) % 16)
    return PD_ERR_UNSUPPORTED;
  if (!aligned(a->k_cache, 16) || !aligned(a->v_cache, 16)) return PD_ERR_UNSUPPORTED;
  if (!aligned(a->q, 2) || (a->out && !aligned(a->out, 2))) return PD_ERR_INVALID_ARG;
  if (a->workspace && !aligned(a->workspace, 256)) return PD_ERR_WORKSPACE;
  return PD_OK;
}

void fill_params(const PdDecodeArgs* a, Params& p) {
  p.q = a->q;
  p.out = a->out;
  p.q_sb = a->q_stride_b;
  p.q_sh = a->q_stride_h;
  p.o_sb = a->out_stride_b;
  p.o_sh = a->out_stride_h;
  p.k = a->k_cache;
  p.v = a->v_cache;
  p.kv_sb = a->kv_stride_block;
  p.kv_st = a->kv_stride_token;
  p.kv_sh = a->kv_stride_head;
  p.k_scale = (const __half*)a->k_scale;
  p.v_scale = (const __half*)a->v_scale;
  p.sc_sb = a->scale_stride_block;
  p.sc_st = a->scale_stride_token;
  p.block_table = a->block_table;
  p.bt_stride = a->block_table_stride;
  p.seq_lens = a->seq_lens;
  p.batch = a->batch;
  p.hq = a->num_q_heads;
  p.hkv = a->num_kv_heads;
  p.d = a->head_dim;
  p.page = a->block_size;
  p.num_blocks = a->num_blocks;
  p.max_blocks = a->max_blocks_per_seq;
  p.group = a->num_q_heads / a->num_kv_heads;
  p.scale_log2 = a->sm_scale * kLog2e;
  p.num_splits = a->num_splits;
  p.block_n = a->block_n ? a->block_n : 64;
  p.part_o = nullptr;
  p.part_lse = nullptr;
  p.res_o = a->result_f32;
  p.res_lse = a->result_lse;
  p.status = a->status;
}

int resolve_sm_count(const PdDecodeArgs* a) {
  return a->sm_count > 0 ? a->sm_count : cached_sm_count();
}

static int select_kernel(const PdDecodeArgs* a) {
  if (a->kernel == PD_KERNEL_SIMPLE) return PD_KERNEL_SIMPLE;
  const int why = stream_supports(a);
  if (why == PD_OK) return PD_KERNEL_STREAM;
  return a->kernel == PD_KERNEL_STREAM ? why : PD_KERNEL_SIMPLE;
}

// Split count the simple kernel will use.
static int simple_splits(const PdDecodeArgs* a, int sm_count) {
  if (a->num_splits > 0) return a->num_splits;
  const int64_t bound64 = (int64_t)a->max_blocks_per_seq * a->block_size;
  int bound = bound64 > INT32_MAX ? INT32_MAX : (int)bound64;
  if (a->max_seq_len > 0 && a->max_seq_len < bound) bound = a->max_seq_len;
  return pd_pick_num_splits(a->batch, a->num_kv_heads, bound, sm_count, a->block_n ? a->block_n : 64);
}

static uint64_t round_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

static uint64_t simple_workspace(const PdDecodeArgs* a, int splits) {
  if (splits <= 1) return 0;
  const uint64_t rows = (uint64_t)a->batch * a->num_q_heads * splits;
  return round_up(rows * a->head_dim * 4, 256) + round_up(rows * 4, 256);
}

template <int KV, bool SCALED>
static cudaError_t launch_simple_d(const Params& p, int io_bf16, dim3 grid, cudaStream_t st) {
#define PD_SIMPLE(DD)                                                                         \
  case DD:                                                                                    \
    if (io_bf16) simple_decode_kernel<KV, DD, true, SCALED><<<grid, kSimpleThreads, 0, st>>>(p); \
    else simple_decode_kernel<KV, DD, false, SCALED><<<grid, kSimpleThreads, 0, st>>>(p);     \
    break;
  switch (p.d) {
    PD_SIMPLE(32)
    PD_SIMPLE(64)
    PD_SIMPLE(128)
    PD_SIMPLE(256)
    default:
      return cudaErrorInvalidValue;
  }
#undef PD_SIMPLE
  return cudaGetLastError();
}

static cudaError_t launch_merge(const MergeParams& m, int io_bf16, cudaStream_t st) {
  if (m.rows <= 0) return cudaSuccess;
  if (io_bf16) merge_kernel<true><<<m.rows, 128, 0, st>>>(m);
  else merge_kernel<false><<<m.rows, 128, 0, st>>>(m);
  return cudaGetLastError();
}

static int run_simple(const PdDecodeArgs* a, Params& p, int sm_count) {
  const int splits = simple_splits(a, sm_count);
  const uint64_t need = simple_workspace(a, splits);
  if (need > 0 && (!a->workspace || a->workspace_bytes < need)) return PD_ERR_WORKSPACE;
  p.num_splits = splits;
  if (splits > 1) {
    const uint64_t rows = (uint64_t)a->batch * a->num_q_heads * splits;
    p.part_o = (float*)a->workspace;
    p.part_lse = (float*)((char*)a->workspace + round_up(rows * a->head_dim * 4, 256));
  }
  if (a->batch == 0) return PD_OK;
  const int gh = a->head_dim <= 128 ? 8 : 4;
  const int chunks = (p.group + gh - 1) / gh;
  const dim3 grid(a->num_kv_heads * chunks, a->batch, splits);
  const cudaStream_t st = (cudaStream_t)a->stream;
  const bool scaled = a->k_scale != nullptr;
  const int bf = a->io_dtype == PD_IO_BF16;
  cudaError_t e;
  switch (a->kv_dtype) {
    case PD_KV_F16: e = launch_simple_d<PD_KV_F16, false>(p, bf, grid, st); break;
    case PD_KV_BF16: e = launch_simple_d<PD_KV_BF16, false>(p, bf, grid, st); break;
    case PD_KV_E5M2:
      e = scaled ? launch_simple_d<PD_KV_E5M2, true>(p, bf, grid, st)
                 : launch_simple_d<PD_KV_E5M2, false>(p, bf, grid, st);
      break;
    default: e = launch_simple_d<PD_KV_I8, true>(p, bf, grid, st); break;
  }
  if (e != cudaSuccess) return PD_ERR_CUDA;
  if (splits > 1) {
    MergeParams m;
    m.part_o = p.part_o;
    m.part_lse = p.part_lse;
    m.rows = a->batch * a->num_q_heads;
    m.parts = splits;
    m.d = a->head_dim;
    m.o_sp = (int64_t)m.rows * a->head_dim;
    m.o_sr = a->head_dim;
    m.l_sp = m.rows;
    m.l_sr = 1;
    m.out = a->out;
    m.dst_sb = a->out_stride_b;
    m.dst_sh = a->out_stride_h;
    m.rows_per_batch = a->num_q_heads;
    m.res_o = a->result_f32;
    m.res_lse = a->result_lse;
    if (launch_merge(m, bf, st) != cudaSuccess) return PD_ERR_CUDA;
  }
  return PD_OK;
}

}  // namespace pd

using namespace pd;

extern "C" {

int pd_abi_version(void) { return PD_ABI_VERSION; }

const char* pd_status_string(int status) {
  switch (status) {
    case PD_OK: return "ok";
    case PD_ERR_INVALID_ARG: return "invalid argument";
    case PD_ERR_UNSUPPORTED: return "unsupported shape, dtype or stride";
    case PD_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case PD_ERR_CUDA: return "CUDA call failed";
    case PD_ERR_TOO_LARGE: return "request needs more scratch than the library's fixed buffer holds";
    default: return "unknown status";
  }
}

int pd_pick_num_splits(int batch, int num_kv_heads, int max_seq_len, int sm_count, int block_n) {
  // Policy for the one-CTA-per-(request, kv head, split) kernel on a 148-SM part: aim for four
  // resident 128-thread CTAs per SM, keep at least four block_n tiles per split so the
  // merge stays a small fraction of the work, never exceed 128 splits.
  if (batch <= 0 || num_kv_heads <= 0 || sm_count <= 0 || block_n <= 0) return 1;
  const long long base = (long long)batch * num_kv_heads;
  const long long target = 4LL * sm_count;
  if (base >= target) return 1;
  const long long want = (target + base - 1) / base;
  const long long useful = (max_seq_len / block_n) / 4;
  long long n = want < useful ? want : useful;
  if (n > 128) n = 128;
  return n < 1 ? 1 : (int)n;
}

int pd_select_kernel(const PdDecodeArgs* args) {
  const int rc = validate(args);
  if (rc != PD_OK) return rc;
  return select_kernel(args);
}

int pd_workspace_bytes(const PdDecodeArgs* args, uint64_t* bytes) {
  if (!bytes) return PD_ERR_INVALID_ARG;
  *bytes = 0;
  const int rc = validate(args);
  if (rc != PD_OK) return rc;
  const int kernel = select_kernel(args);
  if (kernel < 0) return kernel;
  const int sms = resolve_sm_count(args);
  if (sms <= 0) return PD_ERR_CUDA;
  if (kernel == PD_KERNEL_STREAM) {
    *bytes = stream_workspace_bytes(args, sms);
  } else {
    *bytes = simple_workspace(args, simple_splits(args, sms));
  }
  return PD_OK;
}

int pd_counter_bytes(const PdDecodeArgs* args, uint64_t* bytes) {
  if (!bytes) return PD_ERR_INVALID_ARG;
  *bytes = 0;
  const int rc = validate(args);
  if (rc != PD_OK) return rc;
  const int kernel = select_kernel(args);
  if (kernel < 0) return kernel;
  if (kernel != PD_KERNEL_STREAM) return PD_OK;
  const int sms = resolve_sm_count(args);
  if (sms <= 0) return PD_ERR_CUDA;
  *bytes = stream_counter_bytes(args, sms);
  return PD_OK;
}

int pd_decode(const PdDecodeArgs* args) {
  const int rc = validate(args);
  if (rc != PD_OK) return rc;
  const int kernel = select_kernel(args);
  if (kernel < 0) return kernel;
  const int sms = resolve_sm_count(args);
  if (sms <= 0) return PD_ERR_CUDA;
  Params p;
  fill_params(args, p);
  if (kernel == PD_KERNEL_STREAM) return stream_run(args, p, sms);
  return run_simple(args, p, sms);
}

int pd_decode_host(const PdDecodeArgs* args, const PdHostIO* io) {
  const int rc = validate(args);
  if (rc != PD_OK) return rc;
  if (!io || !io->q_host || !io->block_table_host || !io->seq_lens_host || !io->out_host || !args->out)
    return PD_ERR_INVALID_ARG;
  // the staging buffers must be the dense layouts the host arrays have
  if (args->q_stride_h != args->head_dim ||
      args->q_stride_b != (int64_t)args->num_q_heads * args->head_dim ||
      args->out_stride_h != args->head_dim ||
      args->out_stride_b != (int64_t)args->num_q_heads * args->head_dim ||
      args->block_table_stride != args->max_blocks_per_seq)
    return PD_ERR_INVALID_ARG;
  const cudaStream_t st = (cudaStream_t)args->stream;
  const size_t qo = (size_t)args->batch * args->num_q_heads * args->head_dim * 2;
  // PD_FLAG_HOST_DIRECT_*: where the device can address the caller's result (or query) buffer,
  // the kernels use it in place, and the copy behind (or ahead of) the kernel becomes traffic
  // that overlaps the KV stream.
  PdDecodeArgs a = *args;
  a.flags &= ~(PD_FLAG_HOST_DIRECT_OUT | PD_FLAG_HOST_DIRECT_Q | PD_FLAG_HOST_DIRECT_BT);
  bool q_direct = false, out_direct = false, bt_direct = false;
  if (args->flags & PD_FLAG_HOST_DIRECT_BT) {
    void* dbt = device_view_of_host(io->block_table_host);
    if (dbt && ((uintptr_t)dbt % 4) == 0) {
      a.block_table = (const int32_t*)dbt;
      bt_direct = true;
    }
  }
  if (args->flags & PD_FLAG_HOST_DIRECT_Q) {
    void* dq = device_view_of_host(io->q_host);
    if (dq && ((uintptr_t)dq % 16) == 0) {
      a.q = dq;
      a.flags |= PD_FLAG_STAGE_Q;  // whole lines across the bus, not 4-byte pieces
      q_direct = true;
    }
  }
  if (args->flags & PD_FLAG_HOST_DIRECT_OUT) {
    void* dout = device_view_of_host(io->out_host);
    if (dout && ((uintptr_t)dout % 16) == 0) {
      a.out = dout;
      out_direct = true;
    }
  }
  if (args->batch > 0) {
    if ((!q_direct && cudaMemcpyAsync((void*)args->q, io->q_host, qo, cudaMemcpyHostToDevice, st) != cudaSuccess) ||
        (!bt_direct && cudaMemcpyAsync((void*)args->block_table, io->block_table_host,
                                       (size_t)args->batch * args->max_blocks_per_seq * 4, cudaMemcpyHostToDevice,
                                       st) != cudaSuccess) ||
        cudaMemcpyAsync((void*)args->seq_lens, io->seq_lens_host, (size_t)args->batch * 4,
                        cudaMemcpyHostToDevice, st) != cudaSuccess)
      return PD_ERR_CUDA;
  }
  const int drc = pd_decode(&a);
  if (drc != PD_OK) return drc;
  if (args->batch > 0 && !out_direct &&
      cudaMemcpyAsync(io->out_host, args->out, qo, cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return PD_ERR_CUDA;
  return cudaStreamSynchronize(st) == cudaSuccess ? PD_OK : PD_ERR_CUDA;
}

int pd_merge(const PdMergeArgs* a) {
  if (!a || !a->part_out || !a->part_lse) return PD_ERR_INVALID_ARG;
  if (!a->out && !a->result_f32) return PD_ERR_INVALID_ARG;
  if (a->num_parts <= 0 || a->num_rows < 0 || a->head_dim <= 0) return PD_ERR_INVALID_ARG;
  if (a->io_dtype != PD_IO_F16 && a->io_dtype != PD_IO_BF16) return PD_ERR_INVALID_ARG;
  MergeParams m;
  m.part_o = a->part_out;
  m.part_lse = a->part_lse;
  m.o_sp = a->out_stride_p;
  m.o_sr = a->out_stride_row;
  m.l_sp = a->lse_stride_p;
  m.l_sr = a->lse_stride_row;
  m.parts = a->num_parts;
  m.rows = a->num_rows;
  m.d = a->head_dim;
  m.out = a->out;
  m.dst_sb = a->dst_stride_row;
  m.dst_sh = 0;
  m.rows_per_batch = 1;
  m.res_o = a->result_f32;
  m.res_lse = a->result_lse;
  return launch_merge(m, a->io_dtype == PD_IO_BF16, (cudaStream_t)a->stream) == cudaSuccess
             ? PD_OK
             : PD_ERR_CUDA;
}

int pd_gather(const PdGatherArgs* g) {
  if (!g || !g->cache || !g->k_dense || !g->v_dense || g->s_max <= 0) return PD_ERR_INVALID_ARG;
  const PdDecodeArgs* a = g->cache;
  // the gather reads only the cache side of the arguments
  PdDecodeArgs probe = *a;
  static const int dummy = 0;
  if (!probe.q) probe.q = &dummy;
  if (!probe.out) probe.out = (void*)&dummy;
  probe.result_f32 = nullptr;
  probe.result_lse = nullptr;
  const int rc = validate(&probe);
  if (rc != PD_OK) return rc;
  Params p;
  fill_params(a, p);
  const int64_t rows = (int64_t)a->batch * a->num_kv_heads * g->s_max;
  if (rows == 0) return PD_OK;
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  const cudaStream_t st = (cudaStream_t)a->stream;
  __half* kd = (__half*)g->k_dense;
  __half* vd = (__half*)g->v_dense;
  const bool scaled = a->k_scale != nullptr;
#define PD_GATHER(KV, SC)                                                              \
  switch (a->head_dim) {                                                               \
    case 32: gather_kernel<KV, 32, SC><<<blocks, 128, 0, st>>>(p, kd, vd, g->s_max); break;   \
    case 64: gather_kernel<KV, 64, SC><<<blocks, 128, 0, st>>>(p, kd, vd, g->s_max); break;   \
    case 128: gather_kernel<KV, 128, SC><<<blocks, 128, 0, st>>>(p, kd, vd, g->s_max); break; \
    default: gather_kernel<KV, 256, SC><<<blocks, 128, 0, st>>>(p, kd, vd, g->s_max); break;  \
  }
  switch (a->kv_dtype) {
    case PD_KV_F16: PD_GATHER(PD_KV_F16, false) break;
    case PD_KV_BF16: PD_GATHER(PD_KV_BF16, false) break;
    case PD_KV_E5M2:
      if (scaled) { PD_GATHER(PD_KV_E5M2, true) } else { PD_GATHER(PD_KV_E5M2, false) }
      break;
    default: PD_GATHER(PD_KV_I8, true) break;
  }
#undef PD_GATHER
  return cudaGetLastError() == cudaSuccess ? PD_OK : PD_ERR_CUDA;
}

int pd_cache_write(const PdCacheWriteArgs* a) {
  if (!a || !a->key || !a->value || !a->k_cache || !a->v_cache || !a->slot_mapping)
    return PD_ERR_INVALID_ARG;
  if (a->num_tokens < 0 || a->num_kv_heads <= 0 || a->block_size <= 0 || a->num_blocks <= 0)
    return PD_ERR_INVALID_ARG;
  if (a->kv_dtype < PD_KV_F16 || a->kv_dtype > PD_KV_I8) return PD_ERR_INVALID_ARG;
  if (a->io_dtype != PD_IO_F16 && a->io_dtype != PD_IO_BF16) return PD_ERR_INVALID_ARG;
  if ((a->k_scale == nullptr) != (a->v_scale == nullptr)) return PD_ERR_INVALID_ARG;
  if (a->kv_dtype == PD_KV_I8 && !a->k_scale) return PD_ERR_INVALID_ARG;
  if (a->head_dim != 32 && a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256)
    return PD_ERR_UNSUPPORTED;
  // the reference quantises fp16 inputs; 8-bit caches therefore take fp16 keys and values
  if ((a->kv_dtype == PD_KV_I8 || a->kv_dtype == PD_KV_E5M2) && a->io_dtype != PD_IO_F16)
    return PD_ERR_UNSUPPORTED;
  if (a->num_tokens == 0) return PD_OK;
  CacheWriteParams p;
  p.key = a->key;
  p.value = a->value;
  p.in_st = a->in_stride_token;
  p.in_sh = a->in_stride_head;
  p.k_cache = a->k_cache;
  p.v_cache = a->v_cache;
  p.kv_sb = a->kv_stride_block;
  p.kv_st = a->kv_stride_token;
  p.kv_sh = a->kv_stride_head;
  p.k_scale = (__half*)a->k_scale;
  p.v_scale = (__half*)a->v_scale;
  p.sc_sb = a->scale_stride_block;
  p.sc_st = a->scale_stride_token;
  p.slot_mapping = a->slot_mapping;
  p.num_tokens = a->num_tokens;
  p.hkv = a->num_kv_heads;
  p.d = a->head_dim;
  p.page = a->block_size;
  p.num_blocks = a->num_blocks;
  p.status = a->status;
  const int64_t rows = (int64_t)a->num_tokens * a->num_kv_heads;
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  const cudaStream_t st = (cudaStream_t)a->stream;
  const bool bf = a->io_dtype == PD_IO_BF16;
#define PD_CW_D(KV, BF)                                                              \
  switch (a->head_dim) {                                                             \
    case 32: cache_write_kernel<KV, 32, BF><<<blocks, 128, 0, st>>>(p); break;       \
    case 64: cache_write_kernel<KV, 64, BF><<<blocks, 128, 0, st>>>(p); break;       \
    case 128: cache_write_kernel<KV, 128, BF><<<blocks, 128, 0, st>>>(p); break;     \
    default: cache_write_kernel<KV, 256, BF><<<blocks, 128, 0, st>>>(p); break;      \
  }
  switch (a->kv_dtype) {
    case PD_KV_F16:
      if (bf) { PD_CW_D(PD_KV_F16, true) } else { PD_CW_D(PD_KV_F16, false) }
      break;
    case PD_KV_BF16:
      if (bf) { PD_CW_D(PD_KV_BF16, true) } else { PD_CW_D(PD_KV_BF16, false) }
      break;
    case PD_KV_E5M2: PD_CW_D(PD_KV_E5M2, false) break;
    default: PD_CW_D(PD_KV_I8, false) break;
  }
#undef PD_CW_D
  return cudaGetLastError() == cudaSuccess ? PD_OK : PD_ERR_CUDA;
}

uint64_t pd_exchange_bytes(int32_t world, int32_t rows, int32_t head_dim) {
  if (world <= 0 || world > kMaxRanks || rows < 0 || head_dim <= 0) return 0;
  return exchange_bytes(world, rows, head_dim);
}

uint64_t pd_exchange_part_offset(int32_t world, int32_t rows, int32_t head_dim, int32_t parity, int32_t rank) {
  if (world <= 0 || world > kMaxRanks || rows < 0 || head_dim <= 0 || parity < 0 || parity > 1 || rank < 0 ||
      rank >= world)
    return 0;
  return exchange_part_offset(world, rows, head_dim, parity, rank);
}

static int check_exchange(const PdExchangeArgs* a, PeerPointers& peers) {
  if (!a || !a->peer_bufs) return PD_ERR_INVALID_ARG;
  if (a->world <= 0 || a->world > kMaxRanks || a->rank < 0 || a->rank >= a->world) return PD_ERR_INVALID_ARG;
  if (a->rows <= 0 || a->head_dim <= 0 || a->rows_per_batch <= 0) return PD_ERR_INVALID_ARG;
  if (a->phases < 0 || a->phases > (PD_EXCHANGE_SEND | PD_EXCHANGE_MERGE)) return PD_ERR_INVALID_ARG;
  if (a->wait_limit_ns > kExchangeWaitNs) return PD_ERR_INVALID_ARG;
  const bool merging = a->phases == 0 || (a->phases & PD_EXCHANGE_MERGE);
  if (merging && !a->out && !a->result_f32) return PD_ERR_INVALID_ARG;
  if (a->io_dtype != PD_IO_F16 && a->io_dtype != PD_IO_BF16) return PD_ERR_INVALID_ARG;
  for (int r = 0; r < kMaxRanks; ++r) peers.buf[r] = nullptr;
  for (int r = 0; r < a->world; ++r) {
    if (!a->peer_bufs[r] || !aligned(a->peer_bufs[r], 256)) return PD_ERR_INVALID_ARG;
    peers.buf[r] = (unsigned char*)a->peer_bufs[r];
  }
  return PD_OK;
}

// The wait-and-merge launch; `dependent` makes it a programmatic dependent of the kernel ahead
// of it in the stream (its CTAs may be placed while that kernel still runs).
static int launch_exchange_merge(const PdExchangeArgs* a, const PeerPointers& peers, bool dependent) {
  ExchangeMergeParams m;
  m.buf = peers.buf[a->rank];
  m.world = a->world;
  m.rows = a->rows;
  m.d = a->head_dim;
  m.rows_per_batch = a->rows_per_batch;
  m.out = a->out;
  m.dst_sb = a->out_stride_b;
  m.dst_sh = a->out_stride_h;
  m.res_o = a->result_f32;
  m.res_lse = a->result_lse;
  m.status = a->status;
  m.wait_ns = a->wait_limit_ns ? a->wait_limit_ns : kExchangeWaitNs;
  m.after_primary = dependent ? 1 : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a->rows);
  cfg.blockDim = dim3(128);
  cfg.stream = (cudaStream_t)a->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  const cudaError_t e = a->io_dtype == PD_IO_BF16 ? cudaLaunchKernelEx(&cfg, exchange_merge_kernel<true>, m)
                                                  : cudaLaunchKernelEx(&cfg, exchange_merge_kernel<false>, m);
  return e == cudaSuccess ? PD_OK : PD_ERR_CUDA;
}

int pd_exchange_step(const PdExchangeArgs* a) {
  PeerPointers peers;
  const int rc = check_exchange(a, peers);
  if (rc != PD_OK) return rc;
  const bool send = a->phases == 0 || (a->phases & PD_EXCHANGE_SEND);
  const bool merge = a->phases == 0 || (a->phases & PD_EXCHANGE_MERGE);
  if (send) {
    if (!a->local) return PD_ERR_INVALID_ARG;
    if (!aligned(a->local, 4)) return PD_ERR_INVALID_ARG;
    exchange_push_kernel<<<a->world, 256, 0, (cudaStream_t)a->stream>>>(a->local, peers, a->world, a->rank, a->rows,
                                                                         a->head_dim);
    if (cudaGetLastError() != cudaSuccess) return PD_ERR_CUDA;
  }
  return merge ? launch_exchange_merge(a, peers, false) : PD_OK;
}

int pd_decode_exchange(const PdDecodeArgs* d, const PdExchangeArgs* x) {
  const int rc = validate(d, false);
  if (rc != PD_OK) return rc;
  PeerPointers peers;
  const int xrc = check_exchange(x, peers);
  if (xrc != PD_OK) return xrc;
  if (d->kernel == PD_KERNEL_SIMPLE) return PD_ERR_UNSUPPORTED;
  if (d->num_q_heads % d->num_kv_heads) return PD_ERR_INVALID_ARG;
  if (x->rows != d->batch * d->num_q_heads || x->head_dim != d->head_dim || x->rows_per_batch != d->num_q_heads ||
      x->stream != d->stream)
    return PD_ERR_INVALID_ARG;
  const int why = stream_supports(d);
  if (why != PD_OK) return why;
  const int sms = resolve_sm_count(d);
  if (sms <= 0) return PD_ERR_CUDA;
  const bool send = x->phases == 0 || (x->phases & PD_EXCHANGE_SEND);
  const bool merge = x->phases == 0 || (x->phases & PD_EXCHANGE_MERGE);
  if (send) {
    PushTargets push;
    push.peers = peers;
    push.world = x->world;
    push.rank = x->rank;
    push.rows = x->rows;
    Params p;
    fill_params(d, p);
    const int drc = stream_run(d, p, sms, &push);
    if (drc != PD_OK) return drc;
  }
  // as a programmatic dependent only directly behind the decode kernel it belongs to
  return merge ? launch_exchange_merge(x, peers, send) : PD_OK;
}

}  // extern "C"
