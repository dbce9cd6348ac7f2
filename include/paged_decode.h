/*
 * paged_decode.h — C ABI of the B200 (sm_100a) paged-KV grouped-query decode attention.
 *
 * The reference project is pure Python: its decode path is entered through
 * pagedattn/triton_decode.py:285-377 (paged_decode_triton), which launches two Triton
 * kernels.  It has no native interface to mirror, so this header defines the one a binding
 * for that entry point needs: plain pointers, sizes and element strides, an int status on
 * return, no exceptions, no torch types.  Every function is safe to call from several host
 * threads; the library owns no device memory apart from the fixed scratch of pd_decode_static
 * and keeps no mutable state keyed by shapes.
 *
 * Conventions
 *   - all strides are in ELEMENTS of the tensor they describe, not bytes;
 *   - head_dim is contiguous (stride 1) in q, out, k_cache and v_cache;
 *   - k_cache and v_cache share strides (the reference uses K's strides for both,
 *     pagedattn/triton_decode.py:329);
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream;
 *   - return value 0 = success, negative = PD_ERR_*; nothing is launched on error.
 */
#ifndef PAGED_DECODE_B200_H_
#define PAGED_DECODE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PD_ABI_VERSION 2

#if defined(__GNUC__)
#define PD_API __attribute__((visibility("default")))
#else
#define PD_API
#endif

/* status codes */
#define PD_OK 0
#define PD_ERR_INVALID_ARG (-1)   /* null pointer, bad size, bad stride, bad enum      */
#define PD_ERR_UNSUPPORTED (-2)   /* valid request that no compiled kernel serves      */
#define PD_ERR_WORKSPACE (-3)     /* workspace missing, misaligned or too small        */
#define PD_ERR_CUDA (-4)          /* a CUDA runtime/driver call failed                 */
#define PD_ERR_TOO_LARGE (-5)     /* needs more scratch than PD_STATIC_SCRATCH_BYTES   */

/* Size of the library-owned scratch pd_decode_static works in. */
#define PD_STATIC_SCRATCH_BYTES (8u << 20)

/* kv_dtype: element type stored in k_cache / v_cache (pagedattn/config.py:16-31) */
#define PD_KV_F16 0
#define PD_KV_BF16 1
#define PD_KV_E5M2 2
#define PD_KV_I8 3

/* io_dtype: element type of q and out */
#define PD_IO_F16 0
#define PD_IO_BF16 1

/* kernel selector */
#define PD_KERNEL_AUTO 0      /* streaming kernel when it serves the request, else the simple one */
#define PD_KERNEL_SIMPLE 1    /* one CTA per (request, kv head, split); CUDA cores; any stride     */
#define PD_KERNEL_STREAM 2    /* persistent TMA + mbarrier pipeline with tensor-core tiles         */

/* bits of PdDecodeArgs.flags */
#define PD_FLAG_COUNTERS_ZERO 1u /* the caller vouches that the first pd_counter_bytes() bytes of
                                    `workspace` are zero: it zero-filled the workspace once and has
                                    since used it only for calls with these same sizes, dtypes and
                                    split count that completed without PD_DEV_TIMEOUT (every call
                                    leaves its counters at zero).  The per-call clear of the
                                    counters, one memset node ahead of the kernel, is then skipped. */

#define PD_FLAG_EQUAL_TILE_SHARES 2u /* streaming kernel: give every worker the same number of tiles
                                       instead of shares of equal estimated time (a share that
                                       crosses more request boundaries gets fewer tiles); for
                                       A/B measurements */

#define PD_FLAG_HOST_DIRECT_OUT 4u /* pd_decode_host only: out_host is page-locked host memory the device
                                      can address (cudaHostAlloc, cudaHostRegister; what torch's
                                      pin_memory() gives).  The kernels then write the result rows there
                                      themselves, across the bus and while the KV pages stream, instead
                                      of the result being staged in args->out and copied back behind the
                                      kernel.  A pointer the device cannot address is staged as without
                                      the flag. */
#define PD_FLAG_HOST_DIRECT_BT 16u  /* the same for block_table_host: the kernels fetch the entries they
                                      need (one 128-byte read per 32 tiles of a worker) across the bus
                                      instead of the whole padded table being copied ahead of them */
#define PD_FLAG_HOST_DIRECT_Q 8u   /* the same for q_host: the kernels read the query rows from host
                                      memory (implies PD_FLAG_STAGE_Q).  A worker waits for its query
                                      rows when a request starts, and across the bus that wait is
                                      longer: it pays for batches of many requests (the copy it saves
                                      grows with the batch) and costs a few microseconds where a few
                                      long requests are cut over all workers, which then all fetch the
                                      same rows at once. */
#define PD_FLAG_STAGE_Q 32u        /* streaming kernel: a consumer warp first copies the query rows of
                                      its kv head's group into shared memory with 16-byte loads (whole
                                      128-byte lines) and takes its fragments from there, instead of
                                      sixteen 4-byte loads per lane.  Needs the group's rows to be one
                                      dense 16-byte-aligned run and room in shared memory, else it is
                                      ignored.  No faster for q in device memory (0.2 us slower on
                                      cache-resident batches), hence off unless asked for. */

/* bits of the optional device status word (PdDecodeArgs.status) */
#define PD_DEV_BAD_BLOCK 1u   /* a block-table entry was outside [0, num_blocks): page skipped */
#define PD_DEV_TIMEOUT 2u     /* a bounded wait inside a kernel gave up                        */

/*
 * Arguments of one decode step.  Replaces the argument list of paged_decode_triton
 * (pagedattn/triton_decode.py:285-295) plus the fields of PagedKVCache it reads
 * (pagedattn/cache.py:70-80).
 */
typedef struct PdDecodeArgs {
  /* q [batch, num_q_heads, head_dim], out same shape; io_dtype elements */
  const void* q;
  void* out;
  int64_t q_stride_b, q_stride_h;
  int64_t out_stride_b, out_stride_h;

  /* paged cache, NHD: [num_blocks, block_size, num_kv_heads, head_dim] */
  const void* k_cache;
  const void* v_cache;
  int64_t kv_stride_block, kv_stride_token, kv_stride_head;

  /* optional per-(token, head) fp16 scales [num_blocks, block_size, num_kv_heads], head
   * stride 1 (pagedattn/triton_decode.py:145).  Required for PD_KV_I8, optional for
   * PD_KV_E5M2 (an extension: the reference scales int8 only), must be NULL for 16-bit. */
  const void* k_scale;
  const void* v_scale;
  int64_t scale_stride_block, scale_stride_token;

  const int32_t* block_table; /* [batch, max_blocks_per_seq] physical block ids */
  int64_t block_table_stride; /* row stride */
  const int32_t* seq_lens;    /* [batch] tokens held per request; 0 gives a zero output row */

  int32_t batch, num_q_heads, num_kv_heads, head_dim;
  int32_t block_size, num_blocks, max_blocks_per_seq;
  int32_t kv_dtype, io_dtype;

  float sm_scale;     /* multiplies q.k before softmax; never re-derived from head_dim */
  int32_t num_splits; /* >=1: cut every request's KV range into this many block_n-aligned
                         chunks exactly as pagedattn/triton_decode.py:78-82 does;
                         0: automatic (no host sync, seq_lens are never read on the host) */
  int32_t block_n;    /* chunk alignment of the split rule, multiple of block_size; 0 = 64 */
  int32_t kernel;     /* PD_KERNEL_* */
  int32_t sm_count;   /* 0 = query the current device */
  int32_t max_seq_len;/* upper bound on seq_lens if the caller knows one, else 0; only used
                         to choose the automatic split count of PD_KERNEL_SIMPLE */

  /* caller-owned scratch of at least pd_workspace_bytes() bytes, 256-byte aligned.
   * Contents need not be initialised and are meaningless afterwards. */
  void* workspace;
  uint64_t workspace_bytes;

  /* optional extra outputs for merging across devices: the softmax-normalised fp32 result
   * [batch, num_q_heads, head_dim] (contiguous) and its base-2 log-sum-exp
   * [batch, num_q_heads]; -inf marks an empty request.  Both or neither. */
  float* result_f32;
  float* result_lse;

  uint32_t* status; /* optional device word, OR-ed with PD_DEV_* bits; caller zeroes it */
  void* stream;
  uint32_t flags;   /* PD_FLAG_* bits, 0 for none */
} PdDecodeArgs;

/* Host buffers for pd_decode_host. */
typedef struct PdHostIO {
  const void* q_host;             /* contiguous [batch, num_q_heads, head_dim] */
  const int32_t* block_table_host;/* contiguous [batch, max_blocks_per_seq]    */
  const int32_t* seq_lens_host;   /* [batch]                                   */
  void* out_host;                 /* contiguous [batch, num_q_heads, head_dim] */
} PdHostIO;

/* Arguments of the stand-alone log-sum-exp merge.  Replaces _split_reduce_kernel's launch
 * (pagedattn/triton_decode.py:198-240, 368-376) and also merges partial results that
 * came from different GPUs. */
typedef struct PdMergeArgs {
  const float* part_out; /* normalised partial results, addressed [p][row][d] by strides */
  const float* part_lse; /* base-2 log-sum-exp per (p, row); -inf = empty partial         */
  int64_t out_stride_p, out_stride_row; /* d is contiguous                                */
  int64_t lse_stride_p, lse_stride_row;
  int32_t num_parts, num_rows, head_dim; /* rows = batch * num_q_heads */
  void* out;                 /* [num_rows, head_dim] io_dtype, row stride below; may be NULL */
  int64_t dst_stride_row;
  int32_t io_dtype;
  float* result_f32;         /* optional merged fp32 result [num_rows, head_dim] */
  float* result_lse;         /* optional merged lse [num_rows]                   */
  void* stream;
} PdMergeArgs;

/* Arguments of the debug gather: dense fp16 copy of the dequantised pages.  Replaces
 * gather_contiguous (pagedattn/cache.py:187-215); uses the decode kernel's address
 * function, so a bitwise comparison with a CPU gather checks the paging arithmetic. */
typedef struct PdGatherArgs {
  const PdDecodeArgs* cache; /* only the cache, scale, block-table and size fields are read */
  void* k_dense;             /* [batch, num_kv_heads, s_max, head_dim] fp16, contiguous */
  void* v_dense;
  int32_t s_max;
} PdGatherArgs;

/* Arguments of the cache write.  Replaces the call of vLLM's reshape_and_cache_flash in the
 * reference's backend (integration/vllm_backend.py:117-122) and, for 8-bit caches, the
 * quantisation rule of quantize_kv (pagedattn/cache.py:33-48) that the reference applies only
 * when it builds fixtures. */
typedef struct PdCacheWriteArgs {
  const void* key;   /* [num_tokens, num_kv_heads, head_dim] io_dtype, head_dim contiguous */
  const void* value;
  int64_t in_stride_token, in_stride_head;
  void* k_cache;     /* NHD pages, kv_dtype elements */
  void* v_cache;
  int64_t kv_stride_block, kv_stride_token, kv_stride_head;
  void* k_scale;     /* fp16 [num_blocks, block_size, num_kv_heads]; required for PD_KV_I8 */
  void* v_scale;
  int64_t scale_stride_block, scale_stride_token;
  const int64_t* slot_mapping; /* [num_tokens] block * block_size + offset; negative = skip */
  int32_t num_tokens, num_kv_heads, head_dim, block_size, num_blocks;
  int32_t kv_dtype, io_dtype;
  uint32_t* status;  /* optional, PD_DEV_BAD_BLOCK for a slot outside the pool */
  void* stream;
} PdCacheWriteArgs;

/* ABI version of the loaded library (PD_ABI_VERSION it was built with). */
PD_API int pd_abi_version(void);

/* Text for a status code; never NULL. */
PD_API const char* pd_status_string(int status);

/* One decode step on the device: out = softmax(sm_scale * q K^T) V per query head, over the
 * pages the block table names.  Replaces paged_decode_triton
 * (pagedattn/triton_decode.py:285-377). */
PD_API int pd_decode(const PdDecodeArgs* args);

/* The same step for callers that hold q, block_table, seq_lens and out in HOST memory:
 * copies the three inputs into the device buffers named by `args` (which must be large
 * enough), runs pd_decode, copies `out` back and waits for the stream.  With
 * PD_FLAG_HOST_DIRECT_OUT / _BT / _Q in args->flags the kernels use the caller's page-locked
 * out_host / block_table_host / q_host in place instead of that copy.  The KV pages stay where they
 * live, on the device.  No counterpart in the reference, whose callers pass CUDA tensors. */
PD_API int pd_decode_host(const PdDecodeArgs* args, const PdHostIO* io);

/* Bytes of workspace pd_decode needs for these arguments (depends on sizes, dtype, kernel
 * and split count, not on data).  Replaces the reference's shape-keyed global scratch
 * (_Workspace, pagedattn/triton_decode.py:266-282) with caller-owned memory. */
PD_API int pd_workspace_bytes(const PdDecodeArgs* args, uint64_t* bytes);

/* Bytes at the start of the workspace that hold the arrival counters of the streaming kernel's
 * in-kernel merge (0 when the simple kernel would run): what PD_FLAG_COUNTERS_ZERO speaks of.
 * No counterpart in the reference. */
PD_API int pd_counter_bytes(const PdDecodeArgs* args, uint64_t* bytes);

/* Which kernel pd_decode would run: PD_KERNEL_SIMPLE or PD_KERNEL_STREAM, or a negative
 * PD_ERR_* if the arguments are rejected.  Touches no device. */
PD_API int pd_select_kernel(const PdDecodeArgs* args);

/* Split count heuristic for PD_KERNEL_SIMPLE.  Same signature and role as pick_num_splits
 * (pagedattn/triton_decode.py:248-263); the policy is sized for B200's 148 SMs. */
PD_API int pd_pick_num_splits(int batch, int num_kv_heads, int max_seq_len, int sm_count, int block_n);

/* Log-sum-exp merge of partial results (see PdMergeArgs). */
PD_API int pd_merge(const PdMergeArgs* args);

/* Dense dequantised fp16 gather (see PdGatherArgs). */
PD_API int pd_gather(const PdGatherArgs* args);

/* Arguments of the peer exchange: the cross-GPU merge of the KV-range-sharded long-context path
 * done with plain peer stores instead of a collective library.  Nothing in the reference
 * corresponds to it (the reference is single-GPU); the merge arithmetic is that of
 * _split_reduce_kernel (pagedattn/triton_decode.py:221-240) over ranks.  Every rank owns one
 * exchange buffer of pd_exchange_bytes() bytes, zero-filled once, mapped into every peer
 * (e.g. torch symmetric memory); `peer_bufs[r]` is rank r's buffer as seen from this rank.
 * Every value crosses as one indivisible 8-byte word that carries the step's mark beside the
 * float, so nothing is fenced or flagged and a merge uses each word as soon as it is there. */
typedef struct PdExchangeArgs {
  void* const* peer_bufs;  /* host array [world]; entry [rank] is this rank's own buffer */
  int32_t world, rank;     /* world <= 16 */
  const float* local;      /* this rank's partial: rows*head_dim normalised fp32 results, then
                              rows base-2 log-sum-exps (what pd_decode's result_f32/result_lse
                              give when they point into one buffer) */
  int32_t rows, head_dim, rows_per_batch; /* rows = batch * num_q_heads; rows_per_batch = num_q_heads */
  void* out;               /* [batch, num_q_heads, head_dim] io_dtype, strides below; may be NULL */
  int64_t out_stride_b, out_stride_h;
  int32_t io_dtype;
  float* result_f32;       /* optional merged fp32 result [rows, head_dim] */
  float* result_lse;       /* optional merged lse [rows] */
  uint32_t* status;        /* optional device word: PD_DEV_TIMEOUT if a peer's words did not arrive
                              within the wait limit (the merge is then skipped).  After that
                              the ranks may disagree about the step: zero-fill every rank's
                              buffer again before the next step. */
  void* stream;
  int32_t phases;          /* 0 = the whole step; PD_EXCHANGE_SEND = only the part that stores;
                              PD_EXCHANGE_MERGE = only the wait-and-merge.
                              A driver that plays several ranks on one GPU issues every rank's
                              send before any merge, so that no kernel waits for a later one. */
  uint64_t wait_limit_ns;  /* bound of the merge's wait per rank; 0 = one second, never more */
} PdExchangeArgs;

#define PD_EXCHANGE_SEND 1
#define PD_EXCHANGE_MERGE 2

/* Bytes of one rank's exchange buffer (256-byte aligned base expected). */
PD_API uint64_t pd_exchange_bytes(int32_t world, int32_t rows, int32_t head_dim);

/* Byte offset, inside an exchange buffer, of the partial that rank `rank` stores for the step
 * parity `parity` (0 or 1): rows * (head_dim + 1) words of 8 bytes; always a multiple of 256.
 * Exposes the layout for checks. */
PD_API uint64_t pd_exchange_part_offset(int32_t world, int32_t rows, int32_t head_dim, int32_t parity,
                                        int32_t rank);

/* One exchange step: store `local` into every rank's buffer (this rank's own included), then
 * merge the `world` partials that land in this rank's buffer into `out`.  Two kernel launches
 * on `stream`; all ranks must call it once per step. */
PD_API int pd_exchange_step(const PdExchangeArgs* args);

/* Decode and exchange in one: the streaming decode kernel stores every (request, kv head)
 * unit's merged rows into all ranks' exchange buffers itself, as soon as the unit is done, and
 * the wait-and-merge kernel is launched behind it as a programmatic dependent, so its launch
 * overlaps the decode.  Two launches instead of decode + push + merge; nothing in the reference
 * corresponds to it.  `decode` is as for pd_decode with kernel PD_KERNEL_STREAM or AUTO
 * (PD_ERR_UNSUPPORTED when the streaming kernel does not serve it); its `out`, `result_f32` and
 * `result_lse` may all be NULL (the merged result goes to `exchange->out`).  `exchange->local`
 * is not used; rows, head_dim and rows_per_batch must match the decode
 * (rows = batch * num_q_heads). */
PD_API int pd_decode_exchange(const PdDecodeArgs* decode, const PdExchangeArgs* exchange);

/* Failure-path self-test with no counterpart in the reference: runs the kernels' bounded
 * mbarrier wait on a barrier nothing ever completes.  After `limit_ns` (at most one second) the
 * wait gives up, ORs PD_DEV_TIMEOUT into *status (a device word) and the kernel returns
 * normally: the context stays usable.  Lets a host check the give-up path without a fault. */
PD_API int pd_selftest_bounded_wait(uint32_t* status, uint64_t limit_ns, void* stream);

/* Stores this step's keys and values into their cache slots, quantising to the cache's
 * element type with the reference's rules, bit for bit (see PdCacheWriteArgs). */
PD_API int pd_cache_write(const PdCacheWriteArgs* args);

/*
 * pd_decode for callers that have no scratch memory to give and may not allocate any.  It has
 * no counterpart in the reference, whose launcher allocates its split scratch with
 * torch.empty whenever the shape changes.
 *
 * Who needs it: a serving process that handed all free HBM to its KV-page pool at start-up, so
 * a later cudaMalloc would fail; a plugin running on an engine's worker thread where the
 * engine owns the allocator and forbids allocation on the decode path; a host with no
 * allocator of its own at all (a thin C or FFI caller that only holds the pointers it was
 * given).  Such callers pass q, out and the cache exactly as for pd_decode and leave
 * `workspace` NULL (it is ignored); the streaming kernel's arrival counters and partial-result slots live
 * in a fixed PD_STATIC_SCRATCH_BYTES array compiled into the library, which every GPU that
 * loads the library holds until the process exits.
 *
 * Limits and rules:
 *   - only requests the streaming kernel serves (else PD_ERR_UNSUPPORTED), and only those whose
 *     scratch need, pd_workspace_bytes() with kernel = PD_KERNEL_STREAM, is at most
 *     PD_STATIC_SCRATCH_BYTES (else PD_ERR_TOO_LARGE; nothing is launched);
 *   - the first call on each device looks up the array's device address; make that first call
 *     before any stream capture begins;
 *   - all calls on a device share the one array and it keeps the previous call's contents.
 *     The caller clears nothing (each call zeroes the few counters it needs, on its stream,
 *     and writes every other word before reading it), but two calls whose kernels can overlap on the GPU (different streams, or
 *     different host threads on different streams) race on it: keep calls on one stream or
 *     order them yourself;
 *   - no cudaMalloc, cudaFree or other allocating routine is called, host heap included.
 */
PD_API int pd_decode_static(const PdDecodeArgs* args);

#ifdef __cplusplus
}
#endif
#endif /* PAGED_DECODE_B200_H_ */
