/*
 * Minimal C caller of the decode library: builds a tiny paged cache on the device, runs one
 * decode step through pd_decode and prints the first output values.  Nothing here depends on
 * Python or torch; it is what a binding in any language does.
 *
 *   gcc -std=c99 -I include -I /usr/local/cuda/include examples/c_abi_decode.c \
 *       -L paged_decode_attention_b200 -l:libpaged_decode_b200.so -L /usr/local/cuda/lib64 -lcudart \
 *       -Wl,-rpath,$PWD/paged_decode_attention_b200 -o c_abi_decode
 */
#include <cuda_runtime_api.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "paged_decode.h"

/* fp16 bits of a small float, exact for the values used here (multiples of 1/8 below 4). */
static uint16_t half_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const int32_t exp = (int32_t)((u >> 23) & 0xff) - 127 + 15;
  if ((u & 0x7fffffffu) == 0 || exp <= 0) return (uint16_t)sign;
  return (uint16_t)(sign | ((uint32_t)exp << 10) | ((u >> 13) & 0x3ffu));
}

#define CHECK_CUDA(x)                                                        \
  do {                                                                       \
    cudaError_t e_ = (x);                                                    \
    if (e_ != cudaSuccess) {                                                 \
      fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));               \
      return 1;                                                              \
    }                                                                        \
  } while (0)

int main(void) {
  enum { B = 2, HQ = 8, HKV = 2, D = 64, PAGE = 16, NB = 8, MAXB = 4 };
  const int32_t seq_lens[B] = {40, 17};
  const int32_t table[B * MAXB] = {5, 1, 6, 0, 3, 7, 0, 0};
  const size_t kv_elems = (size_t)NB * PAGE * HKV * D, q_elems = (size_t)B * HQ * D;

  uint16_t* h_kv = (uint16_t*)malloc(kv_elems * 2);
  uint16_t* h_q = (uint16_t*)malloc(q_elems * 2);
  for (size_t i = 0; i < kv_elems; ++i) h_kv[i] = half_bits((float)((i * 7) % 17) / 8.f - 1.f);
  for (size_t i = 0; i < q_elems; ++i) h_q[i] = half_bits((float)((i * 5) % 13) / 8.f - 0.75f);

  void *d_k, *d_v, *d_q, *d_out, *d_table, *d_lens, *d_ws = NULL;
  CHECK_CUDA(cudaMalloc(&d_k, kv_elems * 2));
  CHECK_CUDA(cudaMalloc(&d_v, kv_elems * 2));
  CHECK_CUDA(cudaMalloc(&d_q, q_elems * 2));
  CHECK_CUDA(cudaMalloc(&d_out, q_elems * 2));
  CHECK_CUDA(cudaMalloc(&d_table, sizeof table));
  CHECK_CUDA(cudaMalloc(&d_lens, sizeof seq_lens));
  CHECK_CUDA(cudaMemcpy(d_k, h_kv, kv_elems * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(d_v, h_kv, kv_elems * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(d_q, h_q, q_elems * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(d_table, table, sizeof table, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(d_lens, seq_lens, sizeof seq_lens, cudaMemcpyHostToDevice));

  PdDecodeArgs a;
  memset(&a, 0, sizeof a);
  a.q = d_q;
  a.out = d_out;
  a.q_stride_b = a.out_stride_b = HQ * D;
  a.q_stride_h = a.out_stride_h = D;
  a.k_cache = d_k;
  a.v_cache = d_v;
  a.kv_stride_block = PAGE * HKV * D;
  a.kv_stride_token = HKV * D;
  a.kv_stride_head = D;
  a.block_table = (const int32_t*)d_table;
  a.block_table_stride = MAXB;
  a.seq_lens = (const int32_t*)d_lens;
  a.batch = B;
  a.num_q_heads = HQ;
  a.num_kv_heads = HKV;
  a.head_dim = D;
  a.block_size = PAGE;
  a.num_blocks = NB;
  a.max_blocks_per_seq = MAXB;
  a.kv_dtype = PD_KV_F16;
  a.io_dtype = PD_IO_F16;
  a.sm_scale = 0.125f;
  a.kernel = PD_KERNEL_AUTO;

  uint64_t need = 0;
  int rc = pd_workspace_bytes(&a, &need);
  if (rc != PD_OK) {
    fprintf(stderr, "pd_workspace_bytes: %s\n", pd_status_string(rc));
    return 1;
  }
  if (need) CHECK_CUDA(cudaMalloc(&d_ws, need));
  a.workspace = d_ws;
  a.workspace_bytes = need;
  rc = pd_decode(&a);
  if (rc != PD_OK) {
    fprintf(stderr, "pd_decode: %s\n", pd_status_string(rc));
    return 1;
  }
  CHECK_CUDA(cudaDeviceSynchronize());
  uint16_t h_out[4];
  CHECK_CUDA(cudaMemcpy(h_out, d_out, sizeof h_out, cudaMemcpyDeviceToHost));
  printf("kernel %d, scratch %llu bytes, out[0..3] bits: %04x %04x %04x %04x\n", pd_select_kernel(&a),
         (unsigned long long)need, h_out[0], h_out[1], h_out[2], h_out[3]);
  return 0;
}
