// Decode-time head split + rotary embedding: one launch turns the fused q|k|v projection of one
// new token per sequence into the three tensors the layer step takes -- q and k rotated by the
// position's cos/sin (the rotate-half form of the Llama / Qwen2 / Mistral families), v copied --
// and cuts out the (batch, KV head) shard the calling rank owns on the way.  The arithmetic
// rounds where the eager framework ops round (each product and the sum separately, in the
// tensor's own type), so the rows equal those of the reference's call chain
// q_proj/k_proj/v_proj -> view -> apply_rotary_pos_emb (lrqk_attention.py:2254-2275) bit for bit.
#include "common.cuh"

#include <cuda_bf16.h>

namespace lrqk {
namespace {

struct RopeParams {
  const void *qkv, *cos, *sin;
  void *q_out, *k_out, *v_out;
  int32_t q_heads, kv_heads, head_dim, groups;
  int32_t b0, b_count, kvh0, kvh_count;
  int32_t cos_rows;  // bsz, or 1 when all sequences share the position
};

template <typename T> __device__ __forceinline__ float as_float(T x);
template <> __device__ __forceinline__ float as_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float as_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T rounded(float x);
template <> __device__ __forceinline__ float rounded<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 rounded<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// x*c + rot*s with a rounding to T after each of the three operations (no fused multiply-add)
template <typename T> __device__ __forceinline__ T rope_elem(T x, T rot, T c, T s) {
  const T a = rounded<T>(__fmul_rn(as_float(x), as_float(c)));
  const T b = rounded<T>(__fmul_rn(as_float(rot), as_float(s)));
  return rounded<T>(__fadd_rn(as_float(a), as_float(b)));
}

// grid: (local query heads + 2 * local KV heads, b_count); block: head_dim / 2 threads
template <typename T> __global__ void rope_qkv_kernel(RopeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int d = p.head_dim, half = d >> 1, i = threadIdx.x;
  const int hq_local = p.kvh_count * p.groups;
  const int row = blockIdx.x, bl = blockIdx.y, b = p.b0 + bl;
  const int64_t token = (int64_t)b * (p.q_heads + 2 * p.kv_heads) * d;   // this sequence's q|k|v row
  const T *src;
  T *dst;
  bool rotate = true;
  if (row < hq_local) {
    src = (const T *)p.qkv + token + (int64_t)(p.kvh0 * p.groups + row) * d;
    dst = (T *)p.q_out + ((int64_t)bl * hq_local + row) * d;
  } else if (row < hq_local + p.kvh_count) {
    const int h = row - hq_local;
    src = (const T *)p.qkv + token + (int64_t)(p.q_heads + p.kvh0 + h) * d;
    dst = (T *)p.k_out + ((int64_t)bl * p.kvh_count + h) * d;
  } else {
    const int h = row - hq_local - p.kvh_count;
    src = (const T *)p.qkv + token + (int64_t)(p.q_heads + p.kv_heads + p.kvh0 + h) * d;
    dst = (T *)p.v_out + ((int64_t)bl * p.kvh_count + h) * d;
    rotate = false;
  }
  const T lo = src[i], hi = src[i + half];
  if (!rotate) {
    dst[i] = lo;
    dst[i + half] = hi;
    return;
  }
  const int64_t pos_row = p.cos_rows == 1 ? 0 : b;
  const T *c = (const T *)p.cos + pos_row * d, *s = (const T *)p.sin + pos_row * d;
  // rotate_half(x) = [-x[half:], x[:half]]
  dst[i] = rope_elem<T>(lo, rounded<T>(-as_float(hi)), c[i], s[i]);
  dst[i + half] = rope_elem<T>(hi, lo, c[i + half], s[i + half]);
}

}  // namespace
}  // namespace lrqk

extern "C" int lrqk_rope_qkv(const void *qkv, const void *cos, const void *sin, int32_t cos_rows, int32_t dtype,
                             int32_t bsz, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t b0, int32_t b_count,
                             int32_t kvh0, int32_t kvh_count, void *q_out, void *k_out, void *v_out,
                             lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  if (!qkv || !cos || !sin || !q_out || !k_out || !v_out) return LRQK_EINVAL;
  if (cos_rows != 1 && cos_rows != bsz) return LRQK_EINVAL;
  if (bsz <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || q_heads % kv_heads != 0) return LRQK_EINVAL;
  if (b0 < 0 || b_count <= 0 || b0 + b_count > bsz || kvh0 < 0 || kvh_count <= 0 || kvh0 + kvh_count > kv_heads)
    return LRQK_ECAPACITY;
  if (dtype != LRQK_F32 && dtype != LRQK_BF16) return LRQK_EUNSUPPORTED;
  if (head_dim % 2 != 0 || head_dim > 2048 || b_count > 65535) return LRQK_EUNSUPPORTED;
  RopeParams p;
  p.qkv = qkv, p.cos = cos, p.sin = sin;
  p.q_out = q_out, p.k_out = k_out, p.v_out = v_out;
  p.q_heads = q_heads, p.kv_heads = kv_heads, p.head_dim = head_dim, p.groups = q_heads / kv_heads;
  p.b0 = b0, p.b_count = b_count, p.kvh0 = kvh0, p.kvh_count = kvh_count;
  p.cos_rows = cos_rows;
  const dim3 grid((unsigned)(kvh_count * p.groups + 2 * kvh_count), (unsigned)b_count), block((unsigned)(head_dim / 2));
  if (dtype == LRQK_BF16)
    LRQK_CUDA_TRY(launch_dependent(rope_qkv_kernel<__nv_bfloat16>, grid, block, 0, as_stream(stream), 0, p));
  else
    LRQK_CUDA_TRY(launch_dependent(rope_qkv_kernel<float>, grid, block, 0, as_stream(stream), 0, p));
  return LRQK_OK;
}
