// The second half of the rank-r projection step, as device functions shared by the stand-alone
// update kernel (project_update.cu) and the scoring kernel, which applies it itself in the fused
// step (score_topk.cu): the reference's early-exit decision -- a mean over ALL heads of the squared
// change of k_hat (lrqk_attention.py:603-609), re-derived by every CTA from the per-head sums the
// projection kernel left in its workspace -- and, for one head, the line-searched rank-1 step on
// B_Q and B_K (:612-626, :651-665), q_hat and the new row of A_K in the storage dtype.
// One implementation, explicit rounding intrinsics: both callers produce the same bits.
#pragma once

#include "common.cuh"

namespace lrqk {

struct UpdateArgs {
  void *A_K, *B_Q, *B_K;
  const void *q, *k_new;
  const float *ws;       // [N][max_iter][2R+2]: q_hat, k_hat, squared change of k_hat, (pad) per alternation
  void *q_hat;
  int32_t *iters_out;    // optional
  int64_t a_capacity, append_row;
  int32_t q_heads, groups, max_iter, n_heads, head_dim;
  float tol;
};

// The common stopping alternation.  Every thread of the CTA calls; `delta` is shared memory for 8 floats.
// (Sum over the heads: lane-strided partial sums, then the butterfly of warp_sum -- a fixed order.)
template <int R>
__device__ __forceinline__ int update_chosen(const UpdateArgs &u, float *delta) {
  constexpr int W = 2 * R + 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int it = warp; it < u.max_iter && it < 8; it += n_warps) {
    float s = 0.0f;
    for (int hh = lane; hh < u.n_heads; hh += 32) s += u.ws[((int64_t)hh * u.max_iter + it) * W + 2 * R];
    s = warp_sum(s);
    if (lane == 0) delta[it] = s / (float)(u.n_heads * R);
  }
  __syncthreads();
  int c = u.max_iter - 1;
  for (int it = 0; it < u.max_iter && it < 8; ++it) {
    if (delta[it] < u.tol) { c = it; break; }
  }
  return c;
}

// Shared memory update_head needs, in floats: both right factors as fp32, the two projected vectors, scratch.
__host__ __device__ constexpr int update_head_smem_floats(int r, int d) { return 2 * r * d + 2 * r + 16; }

// Head n's update with iterate `chosen`.  Every thread of the CTA calls (blockDim.x >= head_dim).  All threads
// bring B_Q and B_K into shared memory as fp32 (one trip to memory); thread e < head_dim then owns column e of
// both.  `sh`: update_head_smem_floats(R, head_dim) floats, 16-byte aligned.
template <typename T, int R>
__device__ __forceinline__ void update_head(const UpdateArgs &u, int n, int chosen, float *sh) {
  constexpr int W = 2 * R + 2;
  constexpr int EPV = Elt<T>::kPerVec;
  const int D = u.head_dim;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b_idx = n / u.q_heads, h = n % u.q_heads;
  const int kvh = h / u.groups, kv_heads = u.q_heads / u.groups;
  float *Bs = sh;                      // [2][R][D]
  float *hat = sh + 2 * R * D;         // [2][R]
  float *red = hat + 2 * R;            // [2][2][4]
  const float *w = u.ws + ((int64_t)n * u.max_iter + chosen) * W;
  T *Bg[2] = {reinterpret_cast<T *>(u.B_Q) + (int64_t)n * R * D, reinterpret_cast<T *>(u.B_K) + (int64_t)n * R * D};
  const T *xg[2] = {reinterpret_cast<const T *>(u.q) + (int64_t)n * D,
                    reinterpret_cast<const T *>(u.k_new) + ((int64_t)b_idx * kv_heads + kvh) * D};
  // everything this head needs from global memory is asked for in one go: the chosen iterate, this thread's
  // elements of q and k, then the right factors
  const float hat_in = tid < 2 * R ? w[tid] : 0.0f;
  float x_in[2] = {0.0f, 0.0f};
  if (tid < D) { x_in[0] = Elt<T>::to_float(xg[0][tid]); x_in[1] = Elt<T>::to_float(xg[1][tid]); }
  {
    // every load of a thread is requested before the first is stored (up to eight per trip)
    const int per = R * D / EPV, total = 2 * per;
    for (int i0 = tid; i0 < total; i0 += 8 * (int)blockDim.x) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = i0 + k * (int)blockDim.x;
        if (i < total) v[k] = ld16(Bg[i / per] + (int64_t)(i % per) * EPV);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = i0 + k * (int)blockDim.x;
        if (i < total) {
          float f[EPV];
          Elt<T>::unpack(v[k], f);
#pragma unroll
          for (int x = 0; x < EPV; x += 4)
            *reinterpret_cast<float4 *>(Bs + (int64_t)i * EPV + x) = make_float4(f[x], f[x + 1], f[x + 2], f[x + 3]);
        }
      }
    }
  }
  if (tid < 2 * R) hat[tid] = hat_in;
  for (int i = tid + blockDim.x; i < 2 * R; i += blockDim.x) hat[i] = w[i];  // (blockDim.x < 2R: head_dim 64 at rank 64)
  __syncthreads();
  const bool active = tid < D;
  const int e = tid;
  float t[2] = {0.0f, 0.0f};
  if (active) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      float acc = 0.0f;
#pragma unroll 8
      for (int a = 0; a < R; ++a) acc = __fmaf_rn(hat[s * R + a], Bs[(s * R + a) * D + e], acc);
      t[s] = __fsub_rn(acc, x_in[s]);  // (x_hat B - x)[e]
    }
  }
  // |dB|^2 = sum_{a,e} (x_hat[a] t[e])^2 ;  |x_hat dB|^2 = sum_e (sum_a x_hat[a]^2 t[e])^2
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    float n2 = 0.0f, h2 = 0.0f;
    if (active) {
#pragma unroll 8
      for (int a = 0; a < R; ++a) {
        const float dBae = __fmul_rn(hat[s * R + a], t[s]);
        n2 = __fmaf_rn(dBae, dBae, n2);
        h2 = __fmaf_rn(hat[s * R + a], dBae, h2);
      }
    }
    if (warp < 4) {  // the warps that hold columns (head_dim <= 128); idle lanes carry zeros
      n2 = warp_sum(n2);
      const float hh = warp_sum(__fmul_rn(h2, h2));
      if (lane == 0) { red[(s * 2 + 0) * 4 + warp] = n2; red[(s * 2 + 1) * 4 + warp] = hh; }
    }
  }
  __syncthreads();
  if (active) {
    const int col_warps = D / 32;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      float n2 = 0.0f, hh = 0.0f;
      for (int wv = 0; wv < col_warps; ++wv) { n2 = __fadd_rn(n2, red[(s * 2 + 0) * 4 + wv]); hh = __fadd_rn(hh, red[(s * 2 + 1) * 4 + wv]); }
      const float eta = __fdiv_rn(n2, __fadd_rn(hh, 1e-6f));
#pragma unroll 8
      for (int a = 0; a < R; ++a) {
        const float dBae = __fmul_rn(hat[s * R + a], t[s]);
        Bg[s][a * D + e] = Elt<T>::from_float(__fmaf_rn(-eta, dBae, Bs[(s * R + a) * D + e]));
      }
    }
  }
  if (tid < R) {
    reinterpret_cast<T *>(u.q_hat)[(int64_t)n * R + tid] = Elt<T>::from_float(hat[tid]);
    reinterpret_cast<T *>(u.A_K)[((int64_t)n * u.a_capacity + u.append_row) * R + tid] = Elt<T>::from_float(hat[R + tid]);
  }
}

}  // namespace lrqk
