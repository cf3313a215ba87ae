// Hit/miss difference of one head, as a device function: the stand-alone kernel (slot_diff.cu) and
// the tail of the scoring kernel (score_topk.cu) both run it with a 1024-thread CTA.
//
// `wanted` is ascending, so membership of a resident entry is a binary search in shared memory;
// the search also flags the wanted entry as resident.  Two ordered block scans then pair the i-th
// evicted slot (ascending slot number) with the i-th wanted position that is not resident
// (ascending).  The table is updated in place, the mask and per-head miss count are written, and
// the (head, slot, position) triples of the misses are appended to a global list with one atomic
// reservation per CTA.
#pragma once

#include "common.cuh"

namespace lrqk {

constexpr int kDThreads = 1024;

// Bytes of shared memory slot_diff_head needs for k slots: 256 bytes of scratch, then two int32 and two
// byte arrays of k entries.
__host__ __device__ inline size_t slot_diff_smem_bytes(int k) { return 256 + (size_t)k * (2 * sizeof(int32_t) + 2); }

__device__ __forceinline__ uint32_t diff_block_scan(uint32_t v, uint32_t *scratch, uint32_t &total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  uint32_t off = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kDThreads / 32; ++w) {
    const uint32_t s = scratch[w];
    if (w < warp) off += s;
    tot += s;
  }
  __syncthreads();
  total = tot;
  return off + inc - v;
}

// Slot-table entries a thread may fetch ahead of the call (the table does not depend on the selection):
// entries tid, tid + kDThreads, ... of head n, at most kDiffPre of them (k <= kDiffPre * kDThreads).
constexpr int kDiffPre = 4;
struct DiffPre { int32_t v0, v1, v2, v3; bool valid; };  // by value: the entries stay in registers
__device__ __forceinline__ DiffPre slot_diff_preload(int n, const int32_t *table, int k) {
  const int32_t *tab = table + (int64_t)n * k;
  const int t = (int)threadIdx.x;
  DiffPre d;
  d.v0 = t < k ? tab[t] : 0;
  d.v1 = t + kDThreads < k ? tab[t + kDThreads] : 0;
  d.v2 = t + 2 * kDThreads < k ? tab[t + 2 * kDThreads] : 0;
  d.v3 = t + 3 * kDThreads < k ? tab[t + 3 * kDThreads] : 0;
  d.valid = true;
  return d;
}

// One head (n).  `sh` is shared memory of slot_diff_smem_bytes(k) bytes, 16-byte aligned; every
// thread of the kDThreads-thread CTA must call.  `pre` (optional): the thread's table entries as
// slot_diff_preload fetched them (only for k <= kDiffPre * kDThreads).
__device__ __forceinline__ void slot_diff_head(int n, int32_t *table, const int32_t *wanted, uint8_t *mask,
                                               int32_t *miss_count, lrqk_miss *list, int32_t *list_len, int32_t *status,
                                               int k, unsigned char *sh_raw, const DiffPre pre = DiffPre{0, 0, 0, 0, false}) {
  uint32_t *scratch = reinterpret_cast<uint32_t *>(sh_raw);              // [32]
  int32_t *list_base_p = reinterpret_cast<int32_t *>(scratch + 32);      // [1] (+ padding to 64 bytes... 16 words)
  int32_t *w = reinterpret_cast<int32_t *>(sh_raw + 256);                // [k] wanted, ascending
  int32_t *missing = w + k;                                              // [k] wanted-but-not-resident, ascending
  uint8_t *resident = reinterpret_cast<uint8_t *>(missing + k);          // [k] wanted entry already resident
  uint8_t *evict = resident + k;                                         // [k] slot entry no longer wanted
  const int tid = threadIdx.x;
  int32_t *tab = table + (int64_t)n * k;
  const int32_t *wg = wanted + (int64_t)n * k;
  for (int i = tid; i < k; i += kDThreads) { w[i] = __ldcg(wg + i); resident[i] = 0; }
  __syncthreads();
  // (CTA-uniform trip count: the barrier that counts the misses also publishes resident[] and evict[])
  uint32_t n_evict_early = 0;
  for (int i0 = 0, j = 0; i0 < k; i0 += kDThreads, ++j) {
    const int i = i0 + tid;
    bool miss = false;
    if (i < k) {
      // (constant indices keep the preloaded entries in registers)
      const int32_t v = (!pre.valid || j >= kDiffPre) ? tab[i] : (j == 0 ? pre.v0 : j == 1 ? pre.v1 : j == 2 ? pre.v2 : pre.v3);
      int lo = 0, hi = k;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (w[mid] < v) lo = mid + 1; else hi = mid;
      }
      const bool hit = lo < k && w[lo] == v;
      if (hit) resident[lo] = 1;
      evict[i] = hit ? 0 : 1;
      miss = !hit;
    }
    n_evict_early += (uint32_t)__syncthreads_count(miss ? 1 : 0);
  }
  // the reservation in the global miss list is asked for now and read after the two scans below
  if (tid == 0) {
    *list_base_p = n_evict_early ? atomicAdd(list_len, (int32_t)n_evict_early) : 0;
    miss_count[n] = (int32_t)n_evict_early;
  }
  // ordered compaction of the missing wanted entries; each thread owns a contiguous run
  const int per = (k + kDThreads - 1) / kDThreads;
  const int begin = min(k, tid * per), end = min(k, begin + per);
  uint32_t cnt = 0;
  for (int i = begin; i < end; ++i) cnt += resident[i] == 0;
  uint32_t n_missing;
  uint32_t off = diff_block_scan(cnt, scratch, n_missing);
  for (int i = begin; i < end; ++i)
    if (resident[i] == 0) missing[off++] = w[i];
  // ordered scan over the evicted slots
  cnt = 0;
  for (int i = begin; i < end; ++i) cnt += evict[i];
  uint32_t n_evict;
  off = diff_block_scan(cnt, scratch, n_evict);  // the barrier inside also publishes missing[]
  if (tid == 0 && n_evict != n_missing) atomicExch(status, 1);
  __syncthreads();
  const int32_t list_base = *list_base_p;
  const uint32_t usable = n_evict < n_missing ? n_evict : n_missing;
  for (int i = begin; i < end; ++i) {
    uint8_t mk = 0;
    if (evict[i]) {
      if (off < usable) {
        const int32_t pos = missing[off];
        tab[i] = pos;
        lrqk_miss e;
        e.head = n; e.slot = i; e.pos = pos;
        list[list_base + off] = e;
        mk = 1;
      }
      ++off;
    }
    mask[(int64_t)n * k + i] = mk;
  }
}

}  // namespace lrqk
