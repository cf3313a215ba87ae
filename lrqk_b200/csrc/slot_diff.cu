// Hit/miss difference of the wanted set against the resident slot table: one CTA per
// (batch, query head) runs slot_diff_head (slot_diff.cuh).
#include "slot_diff.cuh"

namespace lrqk {
namespace {

__global__ void __launch_bounds__(kDThreads) slot_diff_kernel(int32_t *table, const int32_t *wanted, uint8_t *mask,
                                                             int32_t *miss_count, lrqk_miss *list, int32_t *list_len,
                                                             int32_t *status, int k) {
  extern __shared__ __align__(16) unsigned char sh[];
  pdl_launch_dependents();
  pdl_wait();
  slot_diff_head(blockIdx.x, table, wanted, mask, miss_count, list, list_len, status, k, sh);
}

}  // namespace
}  // namespace lrqk

extern "C" int lrqk_slot_diff(const lrqk_layer *L, const int32_t *wanted, uint8_t *mask, int32_t *miss_count,
                              lrqk_miss *list, int32_t *list_len, int32_t *status, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!wanted || !mask || !miss_count || !list || !list_len || !status || !L->table) return LRQK_EINVAL;
  const size_t smem = slot_diff_smem_bytes(L->k);
  if (smem > 200 * 1024) return LRQK_EUNSUPPORTED;
  static SmemOptIn opt_in;
  if (smem > 48 * 1024) LRQK_CUDA_TRY(opt_in.ensure(slot_diff_kernel, smem));
  LRQK_CUDA_TRY(launch_dependent(slot_diff_kernel, dim3(L->bsz * L->q_heads), dim3(kDThreads), smem, as_stream(stream), 0,
                                 L->table, wanted, mask, miss_count, list, list_len, status, (int)L->k));
  return LRQK_OK;
}
