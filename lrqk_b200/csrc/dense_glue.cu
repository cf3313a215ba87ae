// Element-wise glue of a decoder layer's decode step, fused: residual add + RMSNorm, and SiLU(gate) * up.
//
// The selection path is a handful of launches per layer; the eager framework modules around it (two
// RMSNorms, two residual adds, the SwiGLU activation) are about twenty more, and at one token per step
// every one of them is pure launch latency.  These two kernels stand in for them, rounding where the
// framework's tensor operations round (each product and sum in the tensor's own type), so the rows agree
// with the eager modules to the last bit except where the order of the variance sum differs (one ulp).
#include "common.cuh"

namespace lrqk {
namespace {

constexpr int kGThreads = 256;

template <typename T> __device__ __forceinline__ float to_f(T x) { return Elt<T>::to_float(x); }
template <typename T> __device__ __forceinline__ T rnd(float x) { return Elt<T>::from_float(x); }

struct NormParams {
  const void *x, *delta, *weight;
  void *sum_out, *normed_out;
  int32_t hidden;
  float eps;
};

// One CTA per row: s = x (+ delta), rounded to T; y = weight * T(s * rsqrt(mean(s^2) + eps)).
template <typename T>
__global__ void __launch_bounds__(kGThreads) add_rmsnorm_kernel(NormParams p) {
  extern __shared__ float srow[];   // [hidden] the summed row as fp32
  __shared__ float red[kGThreads / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, h = p.hidden;
  const T *x = reinterpret_cast<const T *>(p.x) + (int64_t)row * h;
  const T *dl = p.delta ? reinterpret_cast<const T *>(p.delta) + (int64_t)row * h : nullptr;
  T *so = p.sum_out ? reinterpret_cast<T *>(p.sum_out) + (int64_t)row * h : nullptr;
  float ss = 0.0f;
  for (int i = tid; i < h; i += kGThreads) {
    float v = to_f(x[i]);
    if (dl) v = to_f(rnd<T>(__fadd_rn(v, to_f(dl[i]))));   // the residual add rounds to T
    if (so) so[i] = rnd<T>(v);
    srow[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int w = 0; w < kGThreads / 32; ++w) tot += red[w];
  const float inv = rsqrtf(tot / (float)h + p.eps);
  const T *wt = reinterpret_cast<const T *>(p.weight);
  T *yo = reinterpret_cast<T *>(p.normed_out) + (int64_t)row * h;
  for (int i = tid; i < h; i += kGThreads) {
    const T n = rnd<T>(__fmul_rn(srow[i], inv));             // hidden_states.to(input_dtype)
    yo[i] = rnd<T>(__fmul_rn(to_f(wt[i]), to_f(n)));         // weight * that
  }
}

// out[r, i] = T(T(silu(gate[r, i])) * up[r, i]) for gate_up [rows, 2 * inter] (gate first, then up).
template <typename T>
__global__ void __launch_bounds__(kGThreads) swiglu_kernel(const T *gate_up, T *out, int32_t inter) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y;
  const int i = blockIdx.x * kGThreads + threadIdx.x;
  if (i >= inter) return;
  const T *g = gate_up + (int64_t)row * 2 * inter;
  const float gv = to_f(g[i]);
  const T act = rnd<T>(gv / (1.0f + expf(-gv)));
  out[(int64_t)row * inter + i] = rnd<T>(__fmul_rn(to_f(act), to_f(g[inter + i])));
}

}  // namespace
}  // namespace lrqk

extern "C" int lrqk_add_rmsnorm(const void *x, const void *delta, const void *weight, float eps, int32_t dtype,
                                int32_t rows, int32_t hidden, void *sum_out, void *normed_out, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  if (!x || !weight || !normed_out || rows <= 0 || hidden <= 0) return LRQK_EINVAL;
  if (dtype != LRQK_F32 && dtype != LRQK_BF16) return LRQK_EUNSUPPORTED;
  if ((size_t)hidden * sizeof(float) > 160 * 1024 || rows > 65535) return LRQK_EUNSUPPORTED;
  NormParams p;
  p.x = x; p.delta = delta; p.weight = weight; p.sum_out = sum_out; p.normed_out = normed_out; p.hidden = hidden; p.eps = eps;
  const size_t smem = (size_t)hidden * sizeof(float);
  static SmemOptIn opt_bf16, opt_f32;
  if (dtype == LRQK_BF16) {
    if (smem > 48 * 1024) LRQK_CUDA_TRY(opt_bf16.ensure(add_rmsnorm_kernel<__nv_bfloat16>, smem));
    LRQK_CUDA_TRY(launch_dependent(add_rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(kGThreads), smem, as_stream(stream), 0, p));
  } else {
    if (smem > 48 * 1024) LRQK_CUDA_TRY(opt_f32.ensure(add_rmsnorm_kernel<float>, smem));
    LRQK_CUDA_TRY(launch_dependent(add_rmsnorm_kernel<float>, dim3(rows), dim3(kGThreads), smem, as_stream(stream), 0, p));
  }
  return LRQK_OK;
}

extern "C" int lrqk_swiglu(const void *gate_up, int32_t dtype, int32_t rows, int32_t inter, void *out, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  if (!gate_up || !out || rows <= 0 || inter <= 0) return LRQK_EINVAL;
  if (dtype != LRQK_F32 && dtype != LRQK_BF16) return LRQK_EUNSUPPORTED;
  if (rows > 65535) return LRQK_EUNSUPPORTED;
  const dim3 grid((unsigned)((inter + kGThreads - 1) / kGThreads), (unsigned)rows);
  if (dtype == LRQK_BF16)
    LRQK_CUDA_TRY(launch_dependent(swiglu_kernel<__nv_bfloat16>, grid, dim3(kGThreads), 0, as_stream(stream), 0,
                                   reinterpret_cast<const __nv_bfloat16 *>(gate_up), reinterpret_cast<__nv_bfloat16 *>(out), inter));
  else
    LRQK_CUDA_TRY(launch_dependent(swiglu_kernel<float>, grid, dim3(kGThreads), 0, as_stream(stream), 0,
                                   reinterpret_cast<const float *>(gate_up), reinterpret_cast<float *>(out), inter));
  return LRQK_OK;
}
