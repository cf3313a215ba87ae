// Row movers: the miss fetch from the page-locked host store into the resident slots, the
// reference's two native gather entry points as device kernels, and the prompt-time copies
// (prompt K|V into the host store, selected rows into the slots).
//
// The host store is read in place over the host link: a warp copies one K|V row with 16-byte
// loads per lane and keeps several rows in flight, so that enough bytes are outstanding to
// cover the link latency.  K goes to K_res, V to V_res -- no staging buffer, no host thread.
#include "common.cuh"

namespace lrqk {
namespace {

constexpr int kGThreads = 256;
constexpr int kRowsInFlight = 4;

// One warp copies `chunks` 16-byte pieces of a row: the first half to dk, the second to dv.
__device__ __forceinline__ void issue_row(const char *src, int chunks, int lane, uint4 (&buf)[4]) {
#pragma unroll
  for (int c = 0; c < 4; ++c)
    if (lane + 32 * c < chunks) buf[c] = ld16(src + (size_t)(lane + 32 * c) * 16);
}
__device__ __forceinline__ void commit_row(char *dk, char *dv, int chunks, int lane, const uint4 (&buf)[4]) {
  const int half = chunks >> 1;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int i = lane + 32 * c;
    if (i < chunks) {
      if (i < half) st16(dk + (size_t)i * 16, buf[c]);
      else st16(dv + (size_t)(i - half) * 16, buf[c]);
    }
  }
}

struct GatherParams {
  const char *host_kv;
  char *K_res, *V_res;
  const lrqk_miss *list;
  const int32_t *list_len;
  int64_t host_capacity;
  int32_t q_heads, groups, kv_heads, slots;  // slots = k + m
  int32_t row_bytes;                         // 2 * d * elt
};

__global__ void __launch_bounds__(kGThreads) miss_gather_kernel(GatherParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * kGThreads + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * kGThreads) >> 5;
  const int total = *p.list_len;
  const int chunks = p.row_bytes >> 4;
  const int half_bytes = p.row_bytes >> 1;
  for (int base = warp_global * kRowsInFlight; base < total; base += n_warps * kRowsInFlight) {
    uint4 buf[kRowsInFlight][4];
    lrqk_miss e[kRowsInFlight];
#pragma unroll
    for (int u = 0; u < kRowsInFlight; ++u) {
      if (base + u < total) {
        e[u] = p.list[base + u];
        if (e[u].pos < 0 || e[u].pos >= p.host_capacity || e[u].slot < 0 || e[u].slot >= p.slots) {
          e[u].head = -1;  // malformed entry: skipped, never dereferenced
          continue;
        }
        const int b = e[u].head / p.q_heads, h = e[u].head % p.q_heads;
        const int64_t row = ((int64_t)b * p.kv_heads + h / p.groups) * p.host_capacity + e[u].pos;
        issue_row(p.host_kv + row * p.row_bytes, chunks, lane, buf[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kRowsInFlight; ++u) {
      if (base + u < total && e[u].head >= 0) {
        const int64_t dst = ((int64_t)e[u].head * p.slots + e[u].slot) * half_bytes;
        commit_row(p.K_res + dst, p.V_res + dst, chunks, lane, buf[u]);
      }
    }
  }
}

// dst[i,:] = src[rows[i],:]
__global__ void __launch_bounds__(kGThreads) index_select_kernel(char *dst, const char *src, const int64_t *rows,
                                                                int64_t n_rows, int64_t row_bytes, int64_t src_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = ((int64_t)blockIdx.x * kGThreads + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * kGThreads) >> 5;
  const int64_t chunks = row_bytes >> 4;
  for (int64_t i = warp_global; i < n_rows; i += n_warps) {
    const int64_t r = rows[i];
    if (r < 0 || r >= src_rows) continue;  // out-of-range rows are skipped, never dereferenced
    const char *s = src + r * row_bytes;
    char *d = dst + i * row_bytes;
    for (int64_t c = lane; c < chunks; c += 32) st16(d + c * 16, ld16(s + c * 16));
  }
}

// ---- take_along_dim_with_mask: count per (b, kv head), exclusive offsets, ordered copy ----------
__global__ void masked_count_kernel(const uint8_t *mask, int64_t per_group, int32_t *counts) {
  // one CTA per (b, kv head); counts[g] = number of set mask bytes of the group
  const uint8_t *mk = mask + (int64_t)blockIdx.x * per_group;
  int c = 0;
  for (int64_t i = threadIdx.x; i < per_group; i += blockDim.x) c += mk[i] != 0;
  __shared__ int red[32];
  c = __reduce_add_sync(0xFFFFFFFFu, c);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
    counts[blockIdx.x] = s;
  }
}

__global__ void masked_offsets_kernel(const int32_t *counts, int64_t n_groups, int64_t *offsets, int64_t *n_out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int64_t run = 0;
    for (int64_t g = 0; g < n_groups; ++g) { offsets[g] = run; run += counts[g]; }
    *n_out = run;
  }
}

__global__ void __launch_bounds__(kGThreads) masked_copy_kernel(char *dst, const char *src, const int64_t *indices,
                                                               const uint8_t *mask, const int64_t *offsets,
                                                               int64_t per_group, int64_t seq_len, int64_t row_bytes) {
  // one CTA per (b, kv head): ordered ranks by a block scan over runs of the mask
  const int64_t g = blockIdx.x;
  const uint8_t *mk = mask + g * per_group;
  const int64_t *idx = indices + g * per_group;
  __shared__ int32_t rank_of[kGThreads + 1];
  __shared__ int32_t run_base;
  if (threadIdx.x == 0) run_base = 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t chunks = row_bytes >> 4;
  for (int64_t t0 = 0; t0 < per_group; t0 += kGThreads) {
    const int64_t i = t0 + threadIdx.x;
    const int flag = i < per_group && mk[i] != 0;
    __syncthreads();
    rank_of[threadIdx.x + 1] = flag;
    __syncthreads();
    if (threadIdx.x == 0) {
      rank_of[0] = run_base;
      for (int j = 1; j <= kGThreads; ++j) rank_of[j] += rank_of[j - 1];
      run_base = rank_of[kGThreads];
    }
    __syncthreads();
    // warp w copies the flagged entries among its 32 positions
    for (int j = 0; j < 32; ++j) {
      const int t = warp * 32 + j;
      const int64_t ii = t0 + t;
      if (ii < per_group && mk[ii] != 0) {
        const int64_t pos = idx[ii];
        if (pos < 0 || pos >= seq_len) continue;
        const char *s = src + (g * seq_len + pos) * row_bytes;
        char *d = dst + (offsets[g] + rank_of[t]) * row_bytes;
        for (int64_t c = lane; c < chunks; c += 32) st16(d + c * 16, ld16(s + c * 16));
      }
    }
  }
}

// ---- prompt K|V into the host store -------------------------------------------------------------
struct PackParams {
  const char *keys, *values;
  char *host_kv;
  int64_t seq_len, host_capacity, host_row;
  int32_t half_bytes;  // d * elt
};
__global__ void __launch_bounds__(kGThreads) kv_pack_kernel(PackParams p, int64_t n_rows) {
  // a warp moves one token: K row then V row, 16 bytes per lane per piece
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = ((int64_t)blockIdx.x * kGThreads + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * kGThreads) >> 5;
  const int chunks = p.half_bytes >> 4;
  for (int64_t i = warp_global; i < n_rows; i += n_warps) {
    const int64_t g = i / p.seq_len, t = i % p.seq_len;
    char *d = p.host_kv + ((g * p.host_capacity + p.host_row + t) * 2) * p.half_bytes;
    const char *sk = p.keys + i * p.half_bytes, *sv = p.values + i * p.half_bytes;
    for (int c = lane; c < chunks; c += 32) {
      st16(d + (size_t)c * 16, ld16(sk + (size_t)c * 16));
      st16(d + p.half_bytes + (size_t)c * 16, ld16(sv + (size_t)c * 16));
    }
  }
}

// ---- selected prompt rows and the last m prompt tokens into the resident slots --------------------
struct FillParams {
  const char *keys, *values;
  char *K_res, *V_res;
  const int32_t *table;
  int32_t *lite_pos;
  int64_t seq_len;
  int32_t q_heads, groups, kv_heads, k, m, half_bytes;
};
__global__ void __launch_bounds__(kGThreads) fill_resident_kernel(FillParams p, int64_t n_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = ((int64_t)blockIdx.x * kGThreads + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * kGThreads) >> 5;
  const int chunks = p.half_bytes >> 4;
  const int slots = p.k + p.m;
  for (int64_t i = warp_global; i < n_rows; i += n_warps) {
    const int n = (int)(i / slots), s = (int)(i % slots);
    const int b = n / p.q_heads, h = n % p.q_heads;
    const int64_t pos = s < p.k ? p.table[(int64_t)n * p.k + s] : p.seq_len - p.m + (s - p.k);
    if (n == 0 && s >= p.k && lane == 0) p.lite_pos[s - p.k] = (int32_t)pos;
    if (pos < 0 || pos >= p.seq_len) continue;
    const int64_t srow = (((int64_t)b * p.kv_heads + h / p.groups) * p.seq_len + pos) * p.half_bytes;
    const int64_t drow = i * p.half_bytes;
    for (int c = lane; c < chunks; c += 32) {
      st16(p.K_res + drow + (size_t)c * 16, ld16(p.keys + srow + (size_t)c * 16));
      st16(p.V_res + drow + (size_t)c * 16, ld16(p.values + srow + (size_t)c * 16));
    }
  }
}

inline int grid_for_rows(int64_t n_rows, int rows_per_warp) {
  const int64_t warps = ceil_div64(n_rows, rows_per_warp);
  const int64_t ctas = ceil_div64(warps, kGThreads / 32);
  const int64_t cap = (int64_t)kNumSMs * 8;
  return (int)(ctas < 1 ? 1 : (ctas > cap ? cap : ctas));
}

}  // namespace
}  // namespace lrqk

extern "C" int lrqk_miss_gather(const lrqk_layer *L, const lrqk_miss *list, const int32_t *list_len,
                                lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!list || !list_len || !L->host_kv || !L->K_res || !L->V_res) return LRQK_EINVAL;
  GatherParams p;
  p.host_kv = reinterpret_cast<const char *>(L->host_kv);
  p.K_res = reinterpret_cast<char *>(L->K_res);
  p.V_res = reinterpret_cast<char *>(L->V_res);
  p.list = list;
  p.list_len = list_len;
  p.host_capacity = L->host_capacity;
  p.q_heads = L->q_heads;
  p.kv_heads = L->kv_heads;
  p.groups = L->q_heads / L->kv_heads;
  p.slots = L->k + L->m;
  p.row_bytes = (int32_t)(2 * L->head_dim * elt_size(L->dtype));
  if (p.row_bytes > 2048) return LRQK_EUNSUPPORTED;
  // the list length is only known on the device: size the grid for the worst case (every slot missed)
  const int64_t worst = (int64_t)L->bsz * L->q_heads * L->k;
  const int grid = grid_for_rows(worst, kRowsInFlight);
  LRQK_CUDA_TRY(launch_dependent(miss_gather_kernel, dim3(grid), dim3(kGThreads), 0, as_stream(stream), 0, p));
  return LRQK_OK;
}

extern "C" int lrqk_d0_indices_select(void *dst, const void *src, const int64_t *rows, int64_t n_rows,
                                      int64_t row_bytes, int64_t src_rows, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  if (n_rows < 0 || row_bytes <= 0 || src_rows < 0) return LRQK_EINVAL;
  if (n_rows == 0) return LRQK_OK;
  if (!dst || !src || !rows) return LRQK_EINVAL;
  if (row_bytes % 16 != 0 || ((uintptr_t)dst | (uintptr_t)src) % 16 != 0) return LRQK_EUNSUPPORTED;
  index_select_kernel<<<grid_for_rows(n_rows, 1), kGThreads, 0, as_stream(stream)>>>(
      reinterpret_cast<char *>(dst), reinterpret_cast<const char *>(src), rows, n_rows, row_bytes, src_rows);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

extern "C" size_t lrqk_take_along_dim_with_mask_workspace_bytes(int64_t bsz, int64_t kv_heads, int64_t groups,
                                                                int64_t k) {
  (void)groups; (void)k;
  if (bsz <= 0 || kv_heads <= 0) return 0;
  return (size_t)(bsz * kv_heads) * (sizeof(int64_t) + sizeof(int32_t)) + 16;
}

extern "C" int lrqk_take_along_dim_with_mask(void *dst, const void *src, const int64_t *indices, const uint8_t *mask,
                                             int64_t bsz, int64_t kv_heads, int64_t seq_len, int64_t groups,
                                             int64_t k, int64_t row_bytes, int64_t *n_out, void *workspace,
                                             lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  if (bsz <= 0 || kv_heads <= 0 || seq_len <= 0 || groups <= 0 || k <= 0 || row_bytes <= 0) return LRQK_EINVAL;
  if (!dst || !src || !indices || !mask || !n_out || !workspace) return LRQK_EINVAL;
  if (row_bytes % 16 != 0 || ((uintptr_t)dst | (uintptr_t)src) % 16 != 0) return LRQK_EUNSUPPORTED;
  const int64_t n_groups = bsz * kv_heads;
  if (n_groups > (1 << 20)) return LRQK_EUNSUPPORTED;
  int64_t *offsets = reinterpret_cast<int64_t *>(workspace);
  int32_t *counts = reinterpret_cast<int32_t *>(offsets + n_groups);
  cudaStream_t s = as_stream(stream);
  masked_count_kernel<<<(int)n_groups, 256, 0, s>>>(mask, groups * k, counts);
  LRQK_LAUNCH_CHECK();
  masked_offsets_kernel<<<1, 32, 0, s>>>(counts, n_groups, offsets, n_out);
  LRQK_LAUNCH_CHECK();
  masked_copy_kernel<<<(int)n_groups, kGThreads, 0, s>>>(reinterpret_cast<char *>(dst),
                                                         reinterpret_cast<const char *>(src), indices, mask, offsets,
                                                         groups * k, seq_len, row_bytes);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

extern "C" int lrqk_kv_pack_host(const lrqk_layer *L, const void *keys, const void *values, int64_t seq_len,
                                 int64_t host_row, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!keys || !values || !L->host_kv || seq_len <= 0 || host_row < 0) return LRQK_EINVAL;
  if (host_row + seq_len > L->host_capacity) return LRQK_ECAPACITY;
  PackParams p;
  p.keys = reinterpret_cast<const char *>(keys);
  p.values = reinterpret_cast<const char *>(values);
  p.host_kv = reinterpret_cast<char *>(L->host_kv);
  p.seq_len = seq_len;
  p.host_capacity = L->host_capacity;
  p.host_row = host_row;
  p.half_bytes = (int32_t)(L->head_dim * elt_size(L->dtype));
  const int64_t n_rows = (int64_t)L->bsz * L->kv_heads * seq_len;
  kv_pack_kernel<<<grid_for_rows(n_rows, 4), kGThreads, 0, as_stream(stream)>>>(p, n_rows);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

extern "C" int lrqk_prefill_fill_resident(const lrqk_layer *L, const void *keys, const void *values, int64_t seq_len,
                                          lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!keys || !values || !L->K_res || !L->V_res || !L->table || !L->lite_pos) return LRQK_EINVAL;
  if (seq_len < L->m) return LRQK_EINVAL;
  FillParams p;
  p.keys = reinterpret_cast<const char *>(keys);
  p.values = reinterpret_cast<const char *>(values);
  p.K_res = reinterpret_cast<char *>(L->K_res);
  p.V_res = reinterpret_cast<char *>(L->V_res);
  p.table = L->table;
  p.lite_pos = L->lite_pos;
  p.seq_len = seq_len;
  p.q_heads = L->q_heads;
  p.kv_heads = L->kv_heads;
  p.groups = L->q_heads / L->kv_heads;
  p.k = L->k;
  p.m = L->m;
  p.half_bytes = (int32_t)(L->head_dim * elt_size(L->dtype));
  const int64_t n_rows = (int64_t)L->bsz * L->q_heads * (L->k + L->m);
  fill_resident_kernel<<<grid_for_rows(n_rows, 2), kGThreads, 0, as_stream(stream)>>>(p, n_rows);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}
