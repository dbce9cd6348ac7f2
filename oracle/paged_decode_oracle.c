/*
 * CPU oracle for paged-KV grouped-query decode attention, plain C with OpenMP.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU baseline of the
 * benchmark.  Nothing in the library links or loads it.
 *
 * Parity status: PINNED against outputs of the unmodified reference stored in
 * tests/golden/golden_v1.npz (see tests/test_oracle_golden.py).
 *
 * It restates pagedattn/reference.py:28-49 (fp32 masked-softmax attention per query head)
 * on top of the page lookup of pagedattn/cache.py:196-214 (position s of request b is token
 * s % PAGE of physical block block_table[b][s / PAGE]) and the dequantisation rule of
 * pagedattn/cache.py:51-62 (fp16(stored), times the per-(token, head) fp16 scale and rounded
 * to fp16 when a scale exists).  Unlike the reference it does not materialise the dense
 * gather first: one (request, kv head) at a time, each stored row is converted once.  The
 * arithmetic per element is the same (fp16 values, fp32 products and sums).
 *
 * Caches are dense NHD arrays [NB][PAGE][Hkv][D]; fp8_e5m2 and bf16 are passed as raw bits.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { PDO_F16 = 0, PDO_BF16 = 1, PDO_E5M2 = 2, PDO_I8 = 3 };

typedef struct PdoCache {
  const void* k_cache;
  const void* v_cache;
  const uint16_t* k_scale; /* fp16 bits or NULL */
  const uint16_t* v_scale;
  const int32_t* block_table;
  const int32_t* seq_lens;
  int32_t batch, num_q_heads, num_kv_heads, head_dim;
  int32_t block_size, num_blocks, max_blocks;
  int32_t kv_dtype;
} PdoCache;

static inline float half_bits_to_float(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}

static inline uint16_t float_to_half_bits(float f) {
  _Float16 x = (_Float16)f; /* round to nearest even */
  uint16_t h;
  memcpy(&h, &x, 2);
  return h;
}

/* fp16 value of one stored element, before any scale (pagedattn/cache.py:55-61). */
static inline uint16_t stored_to_half_bits(const void* base, int64_t idx, int kv_dtype) {
  switch (kv_dtype) {
    case PDO_F16:
      return ((const uint16_t*)base)[idx];
    case PDO_BF16: {
      uint32_t u = (uint32_t)((const uint16_t*)base)[idx] << 16;
      float f;
      memcpy(&f, &u, 4);
      return float_to_half_bits(f);
    }
    case PDO_E5M2:
      return (uint16_t)(((const uint8_t*)base)[idx] << 8);
    default: /* PDO_I8: every int8 is exact in fp16 */
      return float_to_half_bits((float)((const int8_t*)base)[idx]);
  }
}

/* Dequantised fp16 row (as bits) of one (block, token, head). */
static void load_row(const PdoCache* c, const void* store, const uint16_t* scale, int64_t block,
                     int token, int head, uint16_t* row) {
  const int d = c->head_dim;
  const int64_t th = ((int64_t)block * c->block_size + token) * c->num_kv_heads + head;
  const int64_t base = th * d;
  if (scale) {
    const float s = half_bits_to_float(scale[th]);
    for (int i = 0; i < d; ++i) {
      const float x = half_bits_to_float(stored_to_half_bits(store, base + i, c->kv_dtype));
      row[i] = float_to_half_bits(x * s); /* exact fp32 product, one rounding to fp16 */
    }
  } else {
    for (int i = 0; i < d; ++i) row[i] = stored_to_half_bits(store, base + i, c->kv_dtype);
  }
}

/*
 * Dense gather, [B][Hkv][s_max][D] fp16 bits; positions >= seq_len are written as zero.
 * Returns 0, or -1 if a block-table entry is out of range.
 */
int pdo_gather(const PdoCache* c, uint16_t* k_dense, uint16_t* v_dense, int s_max) {
  int bad = 0;
#pragma omp parallel for schedule(dynamic, 1) reduction(| : bad)
  for (int b = 0; b < c->batch; ++b) {
    const int n = c->seq_lens[b];
    for (int h = 0; h < c->num_kv_heads; ++h) {
      for (int s = 0; s < s_max; ++s) {
        const int64_t o = (((int64_t)b * c->num_kv_heads + h) * s_max + s) * c->head_dim;
        if (s >= n) {
          memset(k_dense + o, 0, 2 * (size_t)c->head_dim);
          memset(v_dense + o, 0, 2 * (size_t)c->head_dim);
          continue;
        }
        const int32_t blk = c->block_table[(int64_t)b * c->max_blocks + s / c->block_size];
        if (blk < 0 || blk >= c->num_blocks) {
          bad = 1;
          continue;
        }
        load_row(c, c->k_cache, c->k_scale, blk, s % c->block_size, h, k_dense + o);
        load_row(c, c->v_cache, c->v_scale, blk, s % c->block_size, h, v_dense + o);
      }
    }
  }
  return bad ? -1 : 0;
}

/*
 * out[b][hq][:] = softmax(sm_scale * q[b][hq] . K) V in fp32 over tokens [lo, hi) of each
 * request, where lo = range_lo[b] (0 if NULL) and hi = min(range_hi[b], seq_len) (seq_len if
 * NULL).  If lse is not NULL it receives the base-2 log-sum-exp of the scaled logits
 * (-inf for an empty range, whose output row is zero), matching the split epilogue of
 * pagedattn/triton_decode.py:169-188.  q and out are fp32 [B][Hq][D].
 * Returns 0, -1 for a bad block id, -2 for allocation failure.
 */
int pdo_decode(const PdoCache* c, const float* q, float sm_scale, const int32_t* range_lo,
               const int32_t* range_hi, float* out, float* lse, int num_threads) {
  const int d = c->head_dim, hkv = c->num_kv_heads, hq = c->num_q_heads;
  const int group = hq / hkv;
  int status = 0;
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#else
  (void)num_threads;
#endif
#pragma omp parallel
  {
    uint16_t* row = (uint16_t*)malloc(2 * (size_t)d);
    float* rowf = (float*)malloc(4 * (size_t)d);
    float* logit = NULL;
    size_t logit_cap = 0;
#pragma omp for schedule(dynamic, 1) collapse(2)
    for (int b = 0; b < c->batch; ++b) {
      for (int h = 0; h < hkv; ++h) {
        const int n = c->seq_lens[b];
        const int lo = range_lo ? range_lo[b] : 0;
        int hi = range_hi ? range_hi[b] : n;
        if (hi > n) hi = n;
        float* o = out + ((int64_t)b * hq + (int64_t)h * group) * d;
        memset(o, 0, sizeof(float) * (size_t)group * d);
        if (lo >= hi) {
          if (lse)
            for (int g = 0; g < group; ++g) lse[(int64_t)b * hq + h * group + g] = -INFINITY;
          continue;
        }
        const int len = hi - lo;
        if ((size_t)len * group > logit_cap) {
          free(logit);
          logit_cap = (size_t)len * group;
          logit = (float*)malloc(sizeof(float) * logit_cap);
        }
        if (!row || !rowf || !logit) {
#pragma omp atomic write
          status = -2;
          continue;
        }
        const float* qg = q + ((int64_t)b * hq + (int64_t)h * group) * d;
        int bad = 0;
        /* logits: einsum("bd,bsd->bs") * softmax_scale, pagedattn/reference.py:45 */
        for (int s = 0; s < len; ++s) {
          const int p = lo + s;
          const int32_t blk = c->block_table[(int64_t)b * c->max_blocks + p / c->block_size];
          if (blk < 0 || blk >= c->num_blocks) {
            bad = 1;
            break;
          }
          load_row(c, c->k_cache, c->k_scale, blk, p % c->block_size, h, row);
          for (int i = 0; i < d; ++i) rowf[i] = half_bits_to_float(row[i]);
          for (int g = 0; g < group; ++g) {
            float acc = 0.f;
            for (int i = 0; i < d; ++i) acc += qg[(int64_t)g * d + i] * rowf[i];
            logit[(size_t)g * len + s] = acc * sm_scale;
          }
        }
        if (bad) {
#pragma omp atomic write
          status = -1;
          continue;
        }
        /* softmax over the range, pagedattn/reference.py:46-47 */
        for (int g = 0; g < group; ++g) {
          float* lg = logit + (size_t)g * len;
          float m = lg[0];
          for (int s = 1; s < len; ++s) m = lg[s] > m ? lg[s] : m;
          float sum = 0.f;
          for (int s = 0; s < len; ++s) {
            lg[s] = expf(lg[s] - m);
            sum += lg[s];
          }
          const float inv = 1.f / sum;
          for (int s = 0; s < len; ++s) lg[s] *= inv;
          if (lse) lse[(int64_t)b * hq + h * group + g] = (m + logf(sum)) * 1.4426950408889634f;
        }
        /* out = einsum("bs,bsd->bd"), pagedattn/reference.py:48 */
        for (int s = 0; s < len; ++s) {
          const int p = lo + s;
          const int32_t blk = c->block_table[(int64_t)b * c->max_blocks + p / c->block_size];
          load_row(c, c->v_cache, c->v_scale, blk, p % c->block_size, h, row);
          for (int i = 0; i < d; ++i) rowf[i] = half_bits_to_float(row[i]);
          for (int g = 0; g < group; ++g) {
            const float w = logit[(size_t)g * len + s];
            float* og = o + (int64_t)g * d;
            for (int i = 0; i < d; ++i) og[i] += w * rowf[i];
          }
        }
      }
    }
    free(row);
    free(rowf);
    free(logit);
  }
  return status;
}

int pdo_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
