// Lite-ring write: the step's key/value row goes into ring slot `lite_slot` of every query head
// of its group, its token position into lite_pos, and -- when the write fills the ring -- the
// ring of each KV head is copied in slot order to the host store as K|V rows (posted writes
// over the host link; the page-locked store is addressed directly).
#include "common.cuh"

namespace lrqk {
namespace {

struct LiteParams {
  const char *k_new, *v_new;
  char *K_res, *V_res, *host_kv;
  int32_t *lite_pos;
  int64_t host_capacity, host_row;
  int32_t q_heads, groups, k, m, half_bytes, lite_slot, position, flush_rows;
  int32_t skip_write;  // non-zero: the ring already holds the step's row, only flush
};

__global__ void __launch_bounds__(128) lite_append_kernel(LiteParams p) {
  // one CTA per (batch, kv head)
  pdl_launch_dependents();
  pdl_wait();
  const int g = blockIdx.x;  // b * kv_heads + kvh
  const int kv_heads = p.q_heads / p.groups;
  const int b = g / kv_heads, kvh = g % kv_heads;
  const int chunks = p.half_bytes >> 4;
  const int slots = p.k + p.m;
  const int64_t head0 = (int64_t)b * p.q_heads + (int64_t)kvh * p.groups;
  if (!p.skip_write && g == 0 && threadIdx.x == 0) p.lite_pos[p.lite_slot] = p.position;
  for (int i = threadIdx.x; !p.skip_write && i < chunks * p.groups; i += blockDim.x) {
    const int grp = i / chunks, c = i % chunks;
    const int64_t dst = ((head0 + grp) * slots + p.k + p.lite_slot) * p.half_bytes + (size_t)c * 16;
    st16(p.K_res + dst, ld16(p.k_new + (int64_t)g * p.half_bytes + (size_t)c * 16));
    st16(p.V_res + dst, ld16(p.v_new + (int64_t)g * p.half_bytes + (size_t)c * 16));
  }
  if (p.flush_rows > 0) {
    __syncthreads();  // the row written above is part of the ring that is flushed
    for (int i = threadIdx.x; i < chunks * p.flush_rows; i += blockDim.x) {
      const int j = i / chunks, c = i % chunks;
      const int64_t src = (head0 * slots + p.k + j) * p.half_bytes + (size_t)c * 16;
      char *d = p.host_kv + (((int64_t)g * p.host_capacity + p.host_row + j) * 2) * p.half_bytes + (size_t)c * 16;
      st16(d, ld16(p.K_res + src));
      st16(d + p.half_bytes, ld16(p.V_res + src));
    }
    __threadfence_system();
  }
}

}  // namespace
}  // namespace lrqk

extern "C" int lrqk_lite_append(const lrqk_layer *L, const void *k_new, const void *v_new, int32_t lite_slot,
                                int32_t position, int32_t flush_rows, int64_t host_row, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!k_new || !v_new || !L->K_res || !L->V_res || !L->lite_pos) return LRQK_EINVAL;
  if (lite_slot < 0 || lite_slot >= L->m) return LRQK_ECAPACITY;
  if (flush_rows != 0 && flush_rows != L->m) return LRQK_EINVAL;
  if (flush_rows) {
    if (!L->host_kv || host_row < 0) return LRQK_EINVAL;
    if (host_row + flush_rows > L->host_capacity) return LRQK_ECAPACITY;
  }
  LiteParams p;
  p.k_new = reinterpret_cast<const char *>(k_new);
  p.v_new = reinterpret_cast<const char *>(v_new);
  p.K_res = reinterpret_cast<char *>(L->K_res);
  p.V_res = reinterpret_cast<char *>(L->V_res);
  p.host_kv = reinterpret_cast<char *>(L->host_kv);
  p.lite_pos = L->lite_pos;
  p.host_capacity = L->host_capacity;
  p.host_row = host_row;
  p.q_heads = L->q_heads;
  p.groups = L->q_heads / L->kv_heads;
  p.k = L->k;
  p.m = L->m;
  p.half_bytes = (int32_t)(L->head_dim * elt_size(L->dtype));
  p.lite_slot = lite_slot;
  p.position = position;
  p.flush_rows = flush_rows;
  p.skip_write = 0;
  LRQK_CUDA_TRY(launch_dependent(lite_append_kernel, dim3(L->bsz * L->kv_heads), dim3(128), 0, as_stream(stream), 0, p));
  return LRQK_OK;
}

int lrqk::lite_flush_enqueue(const lrqk_layer *L, int64_t host_row, cudaStream_t stream) {
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!L->K_res || !L->V_res || !L->host_kv || host_row < 0) return LRQK_EINVAL;
  if (host_row + L->m > L->host_capacity) return LRQK_ECAPACITY;
  LiteParams p;
  p.k_new = nullptr; p.v_new = nullptr;
  p.K_res = reinterpret_cast<char *>(L->K_res);
  p.V_res = reinterpret_cast<char *>(L->V_res);
  p.host_kv = reinterpret_cast<char *>(L->host_kv);
  p.lite_pos = L->lite_pos;
  p.host_capacity = L->host_capacity;
  p.host_row = host_row;
  p.q_heads = L->q_heads;
  p.groups = L->q_heads / L->kv_heads;
  p.k = L->k;
  p.m = L->m;
  p.half_bytes = (int32_t)(L->head_dim * elt_size(L->dtype));
  p.lite_slot = 0;
  p.position = 0;
  p.flush_rows = L->m;
  p.skip_write = 1;
  LRQK_CUDA_TRY(launch_dependent(lite_append_kernel, dim3(L->bsz * L->kv_heads), dim3(128), 0, stream, 0, p));
  return LRQK_OK;
}
