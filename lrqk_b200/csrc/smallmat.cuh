// Small dense helpers shared by the projection and the prompt-factorisation kernels.
#pragma once

#include "common.cuh"

namespace lrqk {

// 1/x from the hardware approximation plus one Newton step (about 1 ulp); a full IEEE division
// would sit on the critical path of every elimination column.
__device__ __forceinline__ float fast_rcp(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return fmaf(fmaf(-x, r, 1.0f), r, r);
}

// Inverse of a symmetric positive definite G (R x R in shared memory) into Gi, executed by ONE
// warp with the matrix in registers: lane i owns row i (and i+32 when R = 64) of [G | I].
// Gauss-Jordan elimination without row exchanges.  In step c the pivot row is non-zero exactly in
// columns c .. R+c, so each row keeps only that sliding window of R+1 entries; after every step
// the window is rotated by one so that the pivot column always sits at index 0.  Register
// indices therefore stay compile-time constants inside a ROLLED loop over the columns (straight-
// line elimination code would run once per launch and be bound by instruction fetch), and the
// only communication is the shuffle broadcast of the pivot row.  No barriers.
template <int R>
__device__ __forceinline__ void warp_spd_inverse(const float *G, float *Gi) {
  constexpr int RPL = (R + 31) / 32;
  constexpr unsigned kFull = 0xFFFFFFFFu;
  const int lane = threadIdx.x & 31;
  float w[RPL][R + 1], diag[RPL];
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    const int i = lane + 32 * t;
#pragma unroll
    for (int k = 0; k < R; ++k) w[t][k] = i < R ? G[k * R + i] : 0.0f;  // G is symmetric
    w[t][R] = i == 0 ? 1.0f : 0.0f;                                     // column R: first column of I
    diag[t] = 1.0f;
  }
#pragma unroll 1
  for (int c = 0; c < R; ++c) {
    const int owner = c & 31, slot = c >> 5;
    float src0 = w[0][0];
#pragma unroll
    for (int t = 1; t < RPL; ++t) src0 = slot == t ? w[t][0] : src0;
    const float piv = __shfl_sync(kFull, src0, owner);
    const float rp = fast_rcp(piv);
    float l[RPL];
#pragma unroll
    for (int t = 0; t < RPL; ++t) {
      const bool is_pivot_row = lane == owner && slot == t;
      if (is_pivot_row) diag[t] = piv;
      l[t] = is_pivot_row ? 0.0f : w[t][0] * rp;
    }
#pragma unroll
    for (int k = 1; k <= R; ++k) {
      float src = w[0][k];
#pragma unroll
      for (int t = 1; t < RPL; ++t) src = slot == t ? w[t][k] : src;
      const float pk = __shfl_sync(kFull, src, owner);
#pragma unroll
      for (int t = 0; t < RPL; ++t) w[t][k - 1] = fmaf(-l[t], pk, w[t][k]);  // update and rotate
    }
#pragma unroll
    for (int t = 0; t < RPL; ++t) w[t][R] = lane + 32 * t == c + 1 ? 1.0f : 0.0f;  // next column of I
  }
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    const int i = lane + 32 * t;
    const float rd = fast_rcp(diag[t]);
    if (i < R) {
#pragma unroll
      for (int j = 0; j < R; ++j) Gi[j * R + i] = w[t][j] * rd;  // element (i, j), stored column-wise
    }
  }
  __syncwarp();
}

}  // namespace lrqk
