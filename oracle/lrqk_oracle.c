/*
 * lrqk_oracle.c -- CPU restatement (plain C) of the integer / byte stages of the
 * LRQK decode path.  TEST INFRASTRUCTURE ONLY: nothing in the shipped package
 * may link or call this file; it exists to check the CUDA kernels and to time a
 * CPU baseline.
 *
 * Each function names the place in the reference project whose behaviour it
 * restates (paths are relative to the reference checkout).
 *
 * Build: gcc -O3 -fopenmp -fPIC -shared -o liblrqk_oracle.so lrqk_oracle.c
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Order-preserving map float32 -> uint32 (larger float  <=>  larger key).
 * -0.0f is first folded onto +0.0f so that the two compare equal, as they do
 * under IEEE comparison in the reference's torch.topk. */
static inline uint32_t order_key(float f) {
  uint32_t u;
  if (f == 0.0f) f = 0.0f;
  memcpy(&u, &f, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

static int cmp_u64_desc(const void *a, const void *b) {
  uint64_t x = *(const uint64_t *)a, y = *(const uint64_t *)b;
  return (x < y) - (x > y);
}
static int cmp_i32_asc(const void *a, const void *b) {
  int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
  return (x > y) - (x < y);
}

/*
 * Top-k of each row of `scores` followed by an ascending sort of the chosen
 * positions: lrqk_attention.py:1266-1272 (torch.topk over the sequence axis,
 * then torch.sort of the indices).  torch.topk leaves the order among equal
 * scores unspecified; this restatement fixes it: of equal scores the LOWER
 * position wins.
 *   scores : [n_rows, row_stride] float32, first `c` entries of a row are valid
 *   out    : [n_rows, k] int32 ascending
 * Returns 0, or -1 when k > c.
 */
int oracle_topk_sorted_f32(const float *scores, int64_t n_rows, int64_t c,
                           int64_t row_stride, int32_t k, int32_t *out) {
  if (k > c || k < 0) return -1;
  int rc = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t n = 0; n < n_rows; ++n) {
    uint64_t *comp = (uint64_t *)malloc((size_t)c * sizeof(uint64_t));
    if (!comp) { rc = -2; continue; }
    const float *s = scores + n * row_stride;
    for (int64_t i = 0; i < c; ++i)
      comp[i] = ((uint64_t)order_key(s[i]) << 32) | (uint64_t)(0xFFFFFFFFu - (uint32_t)i);
    qsort(comp, (size_t)c, sizeof(uint64_t), cmp_u64_desc);
    int32_t *o = out + n * (int64_t)k;
    for (int32_t j = 0; j < k; ++j)
      o[j] = (int32_t)(0xFFFFFFFFu - (uint32_t)(comp[j] & 0xFFFFFFFFu));
    qsort(o, (size_t)k, sizeof(int32_t), cmp_i32_asc);
    free(comp);
  }
  return rc;
}

/*
 * Hit/miss difference of the wanted set against the resident slot table:
 * lrqk_attention.py:1275-1315 (`only_indices_in_cpu`; a standalone twin is in
 * cpp_kernel/main_demo.py:123-149).  A resident entry that is still wanted
 * keeps its slot.  The i-th slot (ascending slot number) whose entry is no
 * longer wanted receives the i-th wanted value (in the order it appears in
 * `wanted`) that was not resident -- the effect of the row-major boolean-mask
 * assignment at :1312-1313.
 *   now, wanted : [n_rows, k] int32, each row free of duplicates
 *   updated     : [n_rows, k] int32
 *   mask        : [n_rows, k] uint8, 1 = slot refilled (a miss)
 *   miss_count  : [n_rows] int32 (may be NULL)
 * Returns 0, or -1 if some row has a different number of evicted slots and
 * missing values (only possible with duplicates in the input).
 */
typedef struct { int32_t v; int32_t pos; } vp_t;
static int cmp_vp(const void *a, const void *b) {
  const vp_t *x = (const vp_t *)a, *y = (const vp_t *)b;
  if (x->v != y->v) return (x->v > y->v) - (x->v < y->v);
  return (x->pos > y->pos) - (x->pos < y->pos);
}
static int64_t lower_bound_vp(const vp_t *a, int64_t n, int32_t v) {
  int64_t lo = 0, hi = n;
  while (lo < hi) { int64_t mid = (lo + hi) >> 1; if (a[mid].v < v) lo = mid + 1; else hi = mid; }
  return lo;
}

int oracle_slot_diff(const int32_t *now, const int32_t *wanted, int64_t n_rows, int32_t k,
                     int32_t *updated, uint8_t *mask, int32_t *miss_count) {
  int rc = 0;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < n_rows; ++n) {
    const int32_t *a = now + n * (int64_t)k, *w = wanted + n * (int64_t)k;
    int32_t *u = updated + n * (int64_t)k;
    uint8_t *mk = mask + n * (int64_t)k;
    vp_t *sw = (vp_t *)malloc((size_t)k * sizeof(vp_t));
    uint8_t *wanted_is_resident = (uint8_t *)calloc((size_t)k, 1);
    for (int32_t j = 0; j < k; ++j) { sw[j].v = w[j]; sw[j].pos = j; }
    qsort(sw, (size_t)k, sizeof(vp_t), cmp_vp);
    for (int32_t i = 0; i < k; ++i) {
      int64_t p = lower_bound_vp(sw, k, a[i]);
      int hit = 0;
      for (; p < k && sw[p].v == a[i]; ++p) { wanted_is_resident[sw[p].pos] = 1; hit = 1; }
      mk[i] = (uint8_t)!hit;
      u[i] = a[i];
    }
    int32_t j = 0, misses = 0;
    for (int32_t i = 0; i < k; ++i) {
      if (!mk[i]) continue;
      while (j < k && wanted_is_resident[j]) ++j;
      if (j >= k) { rc = -1; break; }
      u[i] = w[j++];
      ++misses;
    }
    while (j < k && wanted_is_resident[j]) ++j;
    if (j != k) rc = -1;
    if (miss_count) miss_count[n] = misses;
    free(sw); free(wanted_is_resident);
  }
  return rc;
}

/*
 * Linear row numbers of the missed entries into the flattened host K|V store:
 * lrqk_attention.py:71-98.  Entries are listed row-major over
 * (batch, kv_head, group, slot) -- identical to (batch, q_head, slot) -- and a
 * row number is (b * kv_heads + kv_head) * capacity + position (:96-97), where
 * `capacity` is the allocated length of the host store (:113, :1588).
 *   table, mask : [bsz, kv_heads * groups, k]
 *   rows_out    : at least sum(mask) int64
 * Returns the number of rows written.
 */
int64_t oracle_miss_rows(const int32_t *table, const uint8_t *mask, int64_t bsz,
                         int64_t kv_heads, int64_t groups, int32_t k, int64_t capacity,
                         int64_t *rows_out) {
  int64_t m = 0;
  for (int64_t b = 0; b < bsz; ++b)
    for (int64_t h = 0; h < kv_heads; ++h)
      for (int64_t g = 0; g < groups; ++g) {
        const int64_t base = ((b * kv_heads + h) * groups + g) * (int64_t)k;
        for (int32_t s = 0; s < k; ++s)
          if (mask[base + s]) rows_out[m++] = (b * kv_heads + h) * capacity + table[base + s];
      }
  return m;
}

/*
 * dst[i, :] = src[rows[i], :] with one memcpy per row, split over threads:
 * cpp_kernel/take_along_dim_grouped.cpp:133-183 (`d0_indices_select`).
 */
void oracle_gather_rows(uint8_t *dst, const uint8_t *src, const int64_t *rows, int64_t n,
                        int64_t row_bytes) {
#pragma omp parallel for schedule(static) if (n >= 4096)
  for (int64_t i = 0; i < n; ++i)
    memcpy(dst + i * row_bytes, src + rows[i] * row_bytes, (size_t)row_bytes);
}

/*
 * The four-dimensional form of the gather (count, offsets, copy):
 * cpp_kernel/take_along_dim_grouped.cpp:13-124 (`take_along_dim_with_mask`).
 *   src     : [bsz, kv_heads, seq_len, row_bytes] bytes
 *   indices : [bsz, kv_heads, groups, k] int64, mask same shape (uint8)
 *   dst     : [sum(mask), row_bytes]
 * Returns the number of rows copied.
 */
int64_t oracle_take_along_dim_with_mask(uint8_t *dst, const uint8_t *src, const int64_t *indices,
                                        const uint8_t *mask, int64_t bsz, int64_t kv_heads,
                                        int64_t seq_len, int64_t groups, int64_t k,
                                        int64_t row_bytes) {
  int64_t m = 0;
  for (int64_t b = 0; b < bsz; ++b)
    for (int64_t h = 0; h < kv_heads; ++h) {
      const uint8_t *s = src + (b * kv_heads + h) * seq_len * row_bytes;
      const int64_t base = (b * kv_heads + h) * groups * k;
      for (int64_t e = 0; e < groups * k; ++e)
        if (mask[base + e]) {
          memcpy(dst + m * row_bytes, s + indices[base + e] * row_bytes, (size_t)row_bytes);
          ++m;
        }
    }
  return m;
}
