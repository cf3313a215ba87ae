// Prompt factorisation  Q ~ A_Q B_Q,  K ~ A_K B_K  with  A_Q A_K^T ~ Q K^T.
//
// The alternating least squares of the reference touches the long axis (the prompt length S)
// only through products of the form  A^T A,  A^T X  and  X Y  with X in {Q, K}.  After the first
// half-sweep every left factor has the form  A_Q = Q X_Q,  A_K = K X_K  with d x r matrices X, so
// all of those products collapse onto the d x d Gram matrices  S_Q = Q^T Q,  S_K = K^T K:
//     A_Q^T A_Q = X_Q^T S_Q X_Q,   Q^T A_Q = S_Q X_Q,   A_K^T K = X_K^T S_K,  ...
// and the change between sweeps,  mean |A_old - Q X|^2,  is  tr(A_old^T A_old) - 2 tr(X^T Q^T A_old)
// + tr(X^T S_Q X).  The factorisation therefore needs exactly two passes over the prompt:
//   1. gram pass    : per head,  [X | A0]^T [X | A0]  for X = Q and X = K  (S_X, A0^T X, A0^T A0),
//                     split over the prompt and summed in a fixed order;
//   2. algebra      : per head, all sweeps on r x r, r x d and d x d matrices (one CTA per head),
//                     keeping every sweep's result because the stop test of the reference is a
//                     mean over ALL heads and can only be evaluated afterwards;
//   3. apply pass   : the common stopping sweep is derived from the per-head changes, then
//                     A_K = K X_K is written in the storage dtype, together with B_Q, B_K and the
//                     last row of A_Q.
// Arithmetic is fp32 on the stored operands, as in the reference (which up-casts to fp32).
#include "apply_tc.cuh"
#include "common.cuh"
#include "gram_tc.cuh"
#include "smallmat.cuh"

namespace lrqk {
namespace {

constexpr int kFThreads = 256;
constexpr int kGramRows = 32;   // prompt rows staged per tile of the gram pass
constexpr int kApplyRows = 128; // prompt rows per CTA of the apply pass
constexpr int kMaxSweeps = 8;

__host__ __device__ constexpr int pad16(int x) { return (x + 15) / 16 * 16; }

// ---- workspace layout (floats) ------------------------------------------------------------------
struct FactorWs {
  int64_t part;      // [2][N][splits][Wp*Wp]   partial Gram matrices of the two sides
  int64_t head;      // [N][head_stride]        per-head scratch of the algebra kernel
  int64_t sweep;     // [N][sweeps][sweep_stride] per-sweep results
  int64_t status;    // int32 status word of the tensor-core Gram pass
  int64_t total;
  int32_t splits, Wp, head_stride, sweep_stride;
};

__host__ __device__ inline FactorWs factor_ws_layout(int n_heads, int r, int d, int sweeps, int splits) {
  FactorWs w;
  w.splits = splits;
  w.Wp = pad16(r + d);
  // per head: S_Q, S_K (d*d each); G (4 of r*r); C_Q, C_K, B_Q, B_K (r*d each); X_Q, X_K, E, R (d*r each)
  w.head_stride = 2 * d * d + 4 * r * r + 8 * r * d;
  // per sweep: X_Q, X_K (d*r), B_Q, B_K (r*d), ssd_Q, ssd_K (+2 pad)
  w.sweep_stride = 4 * r * d + 4;
  w.part = 0;
  w.head = w.part + (int64_t)2 * n_heads * splits * w.Wp * w.Wp;
  w.sweep = w.head + (int64_t)n_heads * w.head_stride;
  w.status = w.sweep + (int64_t)n_heads * sweeps * w.sweep_stride;  // one word (4 reserved)
  w.total = w.status + 4;
  return w;
}

// ---- 1. gram pass -------------------------------------------------------------------------------
struct GramParams {
  const void *Q, *K;
  const float *A_Q0, *A_K0;
  float *part;
  int64_t seq_len;
  int32_t q_heads, groups, splits, rows_per_split;
};

template <typename T, int R, int D>
__global__ void __launch_bounds__(kFThreads) gram_pass_kernel(GramParams p) {
  constexpr int W = R + D, Wp = pad16(W), TT = Wp / 16;
  constexpr int EPV = Elt<T>::kPerVec;
  const int split = blockIdx.x, n = blockIdx.y, side = blockIdx.z;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int b = n / p.q_heads, h = n % p.q_heads;
  const int kv_heads = p.q_heads / p.groups;
  // side 0: X = Q[b, h], A0 = A_Q0[n];  side 1: X = K[b, h / groups], A0 = A_K0[n]
  const T *X = side == 0 ? reinterpret_cast<const T *>(p.Q) + ((int64_t)n * p.seq_len) * D
                         : reinterpret_cast<const T *>(p.K) + (((int64_t)b * kv_heads + h / p.groups) * p.seq_len) * D;
  const float *A0 = (side == 0 ? p.A_Q0 : p.A_K0) + (int64_t)n * p.seq_len * R;

  __shared__ __align__(16) float zs[kGramRows][Wp];
  float acc[TT][TT];
#pragma unroll
  for (int i = 0; i < TT; ++i)
#pragma unroll
    for (int j = 0; j < TT; ++j) acc[i][j] = 0.0f;
  if constexpr (Wp > W) {  // zero the padding columns once
    for (int i = tid; i < kGramRows * (Wp - W); i += kFThreads) zs[i / (Wp - W)][W + i % (Wp - W)] = 0.0f;
  }

  const int64_t r_begin = (int64_t)split * p.rows_per_split;
  const int64_t r_end = min(p.seq_len, r_begin + p.rows_per_split);
  for (int64_t t0 = r_begin; t0 < r_end; t0 += kGramRows) {
    const int rows = (int)min((int64_t)kGramRows, r_end - t0);
    __syncthreads();
    for (int i = tid; i < kGramRows * D / EPV; i += kFThreads) {
      const int row = i / (D / EPV), c = i % (D / EPV);
      float f[EPV];
      if (row < rows) Elt<T>::unpack(ld16(X + (t0 + row) * D + c * EPV), f);
      else {
#pragma unroll
        for (int e = 0; e < EPV; ++e) f[e] = 0.0f;
      }
#pragma unroll
      for (int e = 0; e < EPV; ++e) zs[row][c * EPV + e] = f[e];
    }
    for (int i = tid; i < kGramRows * R / 4; i += kFThreads) {
      const int row = i / (R / 4), c = i % (R / 4);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < rows) v = *reinterpret_cast<const float4 *>(A0 + (t0 + row) * R + c * 4);
      zs[row][D + c * 4 + 0] = v.x; zs[row][D + c * 4 + 1] = v.y;
      zs[row][D + c * 4 + 2] = v.z; zs[row][D + c * 4 + 3] = v.w;
    }
    __syncthreads();
#pragma unroll 4
    for (int row = 0; row < kGramRows; ++row) {
      float a[TT], c[TT];
#pragma unroll
      for (int i = 0; i < TT; ++i) { a[i] = zs[row][ty * TT + i]; c[i] = zs[row][tx * TT + i]; }
#pragma unroll
      for (int i = 0; i < TT; ++i)
#pragma unroll
        for (int j = 0; j < TT; ++j) acc[i][j] = fmaf(a[i], c[j], acc[i][j]);
    }
  }
  float *out = p.part + ((((int64_t)side * gridDim.y + n) * p.splits) + split) * (int64_t)(Wp * Wp);
#pragma unroll
  for (int i = 0; i < TT; ++i)
#pragma unroll
    for (int j = 0; j < TT; ++j) out[(ty * TT + i) * Wp + tx * TT + j] = acc[i][j];
}

// ---- 2. algebra -----------------------------------------------------------------------------------
// C[m x n] = Add + scale * A[m x k] B[k x n] with arbitrary strides (all operands fp32, any memory);
// every thread of the CTA takes outputs tid, tid + kFThreads, ...  Ends with a barrier.  With scale = 1 the
// sum starts from Add (the unit-weight form's summation order); otherwise the product is summed alone
// and scaled into Add with one fused multiply-add.
__device__ __forceinline__ void mm(float *C, int ldc, const float *A, int a_rs, int a_cs, const float *B, int b_rs,
                                   int b_cs, int m, int n, int k, const float *Add, int add_rs, int add_cs,
                                   float scale = 1.0f) {
  const bool scaled = Add && scale != 1.0f;
  for (int idx = threadIdx.x; idx < m * n; idx += kFThreads) {
    const int i = idx / n, j = idx % n;
    float acc = (Add && !scaled) ? Add[i * add_rs + j * add_cs] : 0.0f;
    const float *ap = A + (int64_t)i * a_rs, *bp = B + (int64_t)j * b_cs;
#pragma unroll 4
    for (int x = 0; x < k; ++x) acc = fmaf(ap[(int64_t)x * a_cs], bp[(int64_t)x * b_rs], acc);
    if (scaled) acc = fmaf(scale, acc, Add[i * add_rs + j * add_cs]);
    C[i * ldc + j] = acc;
  }
  __syncthreads();
}

__device__ __forceinline__ float block_sum(float v, float *red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.0f;
#pragma unroll
  for (int w = 0; w < kFThreads / 32; ++w) s += red[w];
  return s;
}

struct AlgebraParams {
  float *ws;
  FactorWs lay;
  int32_t n_heads, sweeps;
  // Weights of the two reconstruction terms.  With both at 1 a sweep renews A_K from the NEW A_Q
  // (lrqk_attention.py:385-395); otherwise both left factors are renewed from the factors the sweep
  // started with (:266-288) -- the reference's two forms differ in more than the weights.
  float lam_q, lam_k;
};

template <int R, int D>
__global__ void __launch_bounds__(kFThreads) algebra_kernel(AlgebraParams p) {
  constexpr int W = R + D, Wp = pad16(W);
  const int n = blockIdx.x, tid = threadIdx.x, warp = tid >> 5;
  __shared__ __align__(16) float Msm[R * R], Misw[R * R];  // operand / result of the one-warp inversion
  __shared__ float red[kFThreads / 32];

  float *hs = p.ws + p.lay.head + (int64_t)n * p.lay.head_stride;
  float *SQ = hs, *SK = SQ + D * D;
  float *GQ = SK + D * D, *GK = GQ + R * R, *GN = GK + R * R, *Mi = GN + R * R;  // r x r
  float *CQ = Mi + R * R, *CK = CQ + R * D, *BQ = CK + R * D, *BK = BQ + R * D;   // r x d
  float *XQ = BK + R * D, *XK = XQ + D * R, *E = XK + D * R, *RH = E + D * R;     // d x r

  // sum the partial Gram matrices of the prompt splits in split order and cut out the blocks
  for (int side = 0; side < 2; ++side) {
    const float *part = p.ws + p.lay.part + (((int64_t)side * p.n_heads + n) * p.lay.splits) * (int64_t)(Wp * Wp);
    float *S = side == 0 ? SQ : SK, *C = side == 0 ? CQ : CK, *G = side == 0 ? GQ : GK;
    for (int idx = tid; idx < W * W; idx += kFThreads) {
      const int i = idx / W, j = idx % W;
      float s = 0.0f;
      for (int sp = 0; sp < p.lay.splits; ++sp) s += part[(int64_t)sp * Wp * Wp + i * Wp + j];
      if (i < D && j < D) S[i * D + j] = s;                         // X^T X
      else if (i >= D && j < D) C[(i - D) * D + j] = s;             // A0^T X
      else if (i >= D && j >= D) G[(i - D) * R + (j - D)] = s;      // A0^T A0
    }
  }
  __syncthreads();

  // Inverse of a symmetric positive definite r x r matrix in global scratch, through shared memory.
  auto invert = [&](const float *G, float *Gi) {
    for (int i = tid; i < R * R; i += kFThreads) Msm[i] = G[i];
    __syncthreads();
    if (warp == 0) warp_spd_inverse<R>(Msm, Misw);
    __syncthreads();
    for (int i = tid; i < R * R; i += kFThreads) Gi[i] = Misw[(i % R) * R + i / R];  // stored column-wise
    __syncthreads();
  };
  auto trace = [&](const float *G) {
    float v = 0.0f;
    for (int i = tid; i < R; i += kFThreads) v += G[i * R + i];
    return block_sum(v, red);
  };

  const bool unit = p.lam_q == 1.0f && p.lam_k == 1.0f;                       // the reference's dispatch (:790)
  invert(GQ, Mi);
  mm(BQ, D, Mi, R, 1, CQ, D, 1, R, D, R, nullptr, 0, 0);                      // B_Q = G_Q^-1 C_Q
  invert(GK, Mi);
  mm(BK, D, Mi, R, 1, CK, D, 1, R, D, R, nullptr, 0, 0);                      // B_K = G_K^-1 C_K
  for (int sw = 0; sw < p.sweeps; ++sw) {
    float *out = p.ws + p.lay.sweep + ((int64_t)n * p.sweeps + sw) * p.lay.sweep_stride;
    float *oXQ = out, *oXK = oXQ + D * R, *oBQ = oXK + D * R, *oBK = oBQ + R * D, *ossd = oBK + R * D;
    // X_Q = (C_K^T + lam_q B_Q^T)(G_K + lam_q B_Q B_Q^T)^-1
    mm(GN, R, BQ, D, 1, BQ, 1, D, R, R, D, GK, R, 1, p.lam_q);
    invert(GN, Mi);
    for (int i = tid; i < D * R; i += kFThreads) RH[i] = fmaf(p.lam_q, BQ[(i % R) * D + i / R], CK[(i % R) * D + i / R]);
    __syncthreads();
    mm(XQ, R, RH, R, 1, Mi, R, 1, D, R, R, nullptr, 0, 0);
    if (!unit) {
      // X_K = (C_Q^T + lam_k B_K^T)(G_Q + lam_k B_K B_K^T)^-1 from the A_Q the sweep started with
      mm(GN, R, BK, D, 1, BK, 1, D, R, R, D, GQ, R, 1, p.lam_k);
      invert(GN, Mi);
      for (int i = tid; i < D * R; i += kFThreads) RH[i] = fmaf(p.lam_k, BK[(i % R) * D + i / R], CQ[(i % R) * D + i / R]);
      __syncthreads();
      mm(XK, R, RH, R, 1, Mi, R, 1, D, R, R, nullptr, 0, 0);
    }
    mm(E, R, SQ, D, 1, XQ, R, 1, D, R, D, nullptr, 0, 0);                     // Q^T A_Q = S_Q X_Q
    const float tr_old_q = trace(GQ);
    float cross = 0.0f;
    for (int i = tid; i < D * R; i += kFThreads) cross = fmaf(XQ[i], CQ[(i % R) * D + i / R], cross);
    cross = block_sum(cross, red);
    mm(GQ, R, XQ, 1, R, E, R, 1, R, R, D, nullptr, 0, 0);                     // A_Q^T A_Q = X_Q^T S_Q X_Q
    const float ssd_q = tr_old_q - 2.0f * cross + trace(GQ);
    if (unit) {
      // X_K = (Q^T A_Q + B_K^T)(A_Q^T A_Q + B_K B_K^T)^-1 with the new A_Q
      mm(GN, R, BK, D, 1, BK, 1, D, R, R, D, GQ, R, 1);
      invert(GN, Mi);
      for (int i = tid; i < D * R; i += kFThreads) RH[i] = E[i] + BK[(i % R) * D + i / R];
    }
    for (int i = tid; i < D * R; i += kFThreads) oXQ[i] = XQ[i];
    __syncthreads();
    for (int i = tid; i < R * D; i += kFThreads) CQ[i] = E[(i % D) * R + i / D];  // A_Q^T Q = E^T
    if (unit) mm(XK, R, RH, R, 1, Mi, R, 1, D, R, R, nullptr, 0, 0);
    else __syncthreads();
    mm(E, R, SK, D, 1, XK, R, 1, D, R, D, nullptr, 0, 0);                     // K^T A_K = S_K X_K
    const float tr_old_k = trace(GK);
    cross = 0.0f;
    for (int i = tid; i < D * R; i += kFThreads) cross = fmaf(XK[i], CK[(i % R) * D + i / R], cross);
    cross = block_sum(cross, red);
    mm(GK, R, XK, 1, R, E, R, 1, R, R, D, nullptr, 0, 0);                     // A_K^T A_K
    const float ssd_k = tr_old_k - 2.0f * cross + trace(GK);
    for (int i = tid; i < R * D; i += kFThreads) CK[i] = E[(i % D) * R + i / D];  // A_K^T K
    for (int i = tid; i < D * R; i += kFThreads) oXK[i] = XK[i];
    __syncthreads();
    // right factors of the new left factors (also the starting point of the next sweep)
    invert(GQ, Mi);
    mm(BQ, D, Mi, R, 1, CQ, D, 1, R, D, R, nullptr, 0, 0);
    invert(GK, Mi);
    mm(BK, D, Mi, R, 1, CK, D, 1, R, D, R, nullptr, 0, 0);
    for (int i = tid; i < R * D; i += kFThreads) { oBQ[i] = BQ[i]; oBK[i] = BK[i]; }
    if (tid == 0) { ossd[0] = ssd_q; ossd[1] = ssd_k; }
    __syncthreads();
  }
}

// ---- 3. apply pass --------------------------------------------------------------------------------
struct ApplyParams {
  const void *Q, *K;
  void *A_K, *B_Q, *B_K, *a_q_last;
  const float *ws;
  FactorWs lay;
  int32_t *sweeps_out;
  int64_t seq_len, a_capacity;
  int32_t q_heads, groups, n_heads, sweeps;
  float tol;
  int32_t rows_elsewhere;  // non-zero: the rows of A_K are written by the tensor-core apply pass
};

template <typename T, int R, int D>
__global__ void __launch_bounds__(kFThreads) apply_kernel(ApplyParams p) {
  constexpr int CPT = R / 2;  // output columns per thread (two threads share a prompt row)
  const int tile = blockIdx.x, n = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = n / p.q_heads, h = n % p.q_heads, kv_heads = p.q_heads / p.groups;
  __shared__ __align__(16) float Xs[D * R];
  __shared__ float delta[2][kMaxSweeps];
  __shared__ int chosen;

  // stopping sweep: first sweep whose mean squared change of both left factors is below tol
  for (int i = warp; i < 2 * p.sweeps; i += kFThreads / 32) {
    const int sw = i >> 1, which = i & 1;
    float s = 0.0f;
    for (int hh = lane; hh < p.n_heads; hh += 32)
      s += p.ws[p.lay.sweep + ((int64_t)hh * p.sweeps + sw) * p.lay.sweep_stride + 4 * R * D + which];
    s = warp_sum(s);
    if (lane == 0) delta[which][sw] = s / ((float)p.n_heads * (float)p.seq_len * (float)R);
  }
  __syncthreads();
  if (tid == 0) {
    int c = p.sweeps - 1;
    for (int sw = 0; sw < p.sweeps; ++sw)
      if (fmaxf(delta[0][sw], delta[1][sw]) < p.tol) { c = sw; break; }
    chosen = c;
    if (n == 0 && tile == 0 && p.sweeps_out) *p.sweeps_out = c + 1;
  }
  __syncthreads();
  const float *res = p.ws + p.lay.sweep + ((int64_t)n * p.sweeps + chosen) * p.lay.sweep_stride;
  const float *XQ = res, *XK = XQ + D * R, *BQf = XK + D * R, *BKf = BQf + R * D;
  for (int i = tid; i < D * R; i += kFThreads) Xs[i] = XK[i];
  __syncthreads();

  // A_K rows of this tile: thread (row, half) forms R/2 columns of  K[row] X_K
  const T *Kh = reinterpret_cast<const T *>(p.K) + (((int64_t)b * kv_heads + h / p.groups) * p.seq_len) * D;
  T *AKh = reinterpret_cast<T *>(p.A_K) + (int64_t)n * p.a_capacity * R;
  const int64_t row = (int64_t)tile * kApplyRows + tid / 2;
  const int c0 = (tid % 2) * CPT;
  if (row < p.seq_len && !p.rows_elsewhere) {
    float acc[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) acc[c] = 0.0f;
    constexpr int EPV = Elt<T>::kPerVec;
    for (int e0 = 0; e0 < D; e0 += EPV) {
      float kf[EPV];
      Elt<T>::unpack(ld16(Kh + row * D + e0), kf);
#pragma unroll
      for (int e = 0; e < EPV; ++e) {
#pragma unroll
        for (int c = 0; c < CPT; c += 4) {
          const float4 x = *reinterpret_cast<const float4 *>(Xs + (e0 + e) * R + c0 + c);
          acc[c] = fmaf(kf[e], x.x, acc[c]); acc[c + 1] = fmaf(kf[e], x.y, acc[c + 1]);
          acc[c + 2] = fmaf(kf[e], x.z, acc[c + 2]); acc[c + 3] = fmaf(kf[e], x.w, acc[c + 3]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) AKh[row * R + c0 + c] = Elt<T>::from_float(acc[c]);
  }
  if (tile == 0) {
    T *BQo = reinterpret_cast<T *>(p.B_Q) + (int64_t)n * R * D, *BKo = reinterpret_cast<T *>(p.B_K) + (int64_t)n * R * D;
    for (int i = tid; i < R * D; i += kFThreads) {
      BQo[i] = Elt<T>::from_float(BQf[i]);
      BKo[i] = Elt<T>::from_float(BKf[i]);
    }
    // last row of A_Q = Q[S-1] X_Q
    const T *qlast = reinterpret_cast<const T *>(p.Q) + ((int64_t)n * p.seq_len + (p.seq_len - 1)) * D;
    if (tid < R) {
      float acc = 0.0f;
      for (int e = 0; e < D; ++e) acc = fmaf(Elt<T>::to_float(qlast[e]), XQ[e * R + tid], acc);
      reinterpret_cast<T *>(p.a_q_last)[(int64_t)n * R + tid] = Elt<T>::from_float(acc);
    }
  }
}

int plan_gram_splits(int n_heads, int64_t seq_len) {
  int splits = (4 * kNumSMs + 2 * n_heads - 1) / (2 * n_heads);
  if (splits < 1) splits = 1;
  const int64_t max_by_rows = (seq_len + 1023) / 1024;
  if (splits > max_by_rows) splits = (int)max_by_rows;
  if (splits > 64) splits = 64;
  return splits;
}

template <typename T, int R, int D>
int run(const lrqk_layer *L, const void *Q, const void *K, float *A_Q, float *A_K_init, int64_t seq_len, int sweeps,
        float tol, void *a_q_last, int32_t *sweeps_out, float *ws, cudaStream_t stream) {
  const int n_heads = L->bsz * L->q_heads;
  const int splits = plan_gram_splits(n_heads, seq_len);
  const FactorWs lay = factor_ws_layout(n_heads, R, D, sweeps, splits);
  const int groups = L->q_heads / L->kv_heads;
  bool on_tensor_cores = false;
  if constexpr (sizeof(T) == 2 && D == 128) {
    // bf16 prompts: tcgen05 Gram pass.  It rounds the initial left factors to bf16 (they are a
    // random or column-sampled starting point; the same rounded values enter every product).
    GramTcArgs ta;
    ta.Q = Q; ta.K = K; ta.A_Q0 = A_Q; ta.A_K0 = A_K_init; ta.part = ws + lay.part;
    ta.status = reinterpret_cast<int32_t *>(ws + lay.status);
    ta.seq_len = seq_len; ta.bsz = L->bsz; ta.q_heads = L->q_heads; ta.kv_heads = L->kv_heads; ta.head_dim = D; ta.r = R;
    ta.splits = splits;
    ta.rows_per_split = (int32_t)(ceil_div64(ceil_div64(seq_len, splits), gram_tc_tile_rows()) * gram_tc_tile_rows());
    LRQK_CUDA_TRY(cudaMemsetAsync(ta.status, 0, sizeof(int32_t), stream));
    const int rc = launch_gram_tc(ta, stream);
    if (rc == LRQK_OK) on_tensor_cores = true;
    else if (rc != LRQK_EUNSUPPORTED) return rc;
  }
  if (!on_tensor_cores) {
    GramParams gp;
    gp.Q = Q; gp.K = K; gp.A_Q0 = A_Q; gp.A_K0 = A_K_init; gp.part = ws + lay.part;
    gp.seq_len = seq_len; gp.q_heads = L->q_heads; gp.groups = groups; gp.splits = splits;
    gp.rows_per_split = (int32_t)(ceil_div64(ceil_div64(seq_len, splits), kGramRows) * kGramRows);
    gram_pass_kernel<T, R, D><<<dim3(splits, n_heads, 2), kFThreads, 0, stream>>>(gp);
    LRQK_LAUNCH_CHECK();
  }
  AlgebraParams ap;
  ap.ws = ws; ap.lay = lay; ap.n_heads = n_heads; ap.sweeps = sweeps;
  ap.lam_q = L->weights[0]; ap.lam_k = L->weights[1];  // lambda_Q, lambda_K (:1435-1436)
  algebra_kernel<R, D><<<n_heads, kFThreads, 0, stream>>>(ap);
  LRQK_LAUNCH_CHECK();
  ApplyParams pp;
  pp.Q = Q; pp.K = K; pp.A_K = L->A_K; pp.B_Q = L->B_Q; pp.B_K = L->B_K; pp.a_q_last = a_q_last;
  pp.ws = ws; pp.lay = lay; pp.sweeps_out = sweeps_out; pp.seq_len = seq_len; pp.a_capacity = L->a_capacity;
  pp.q_heads = L->q_heads; pp.groups = groups; pp.n_heads = n_heads; pp.sweeps = sweeps; pp.tol = tol;
  pp.rows_elsewhere = 0;
  if constexpr (sizeof(T) == 2 && D == 128) {
    // bf16 prompts: A_K = K X_K on the tensor cores (X_K rounded to bf16); the SIMT kernel then only
    // writes B_Q, B_K and the last row of A_Q
    if (on_tensor_cores) {
      ApplyTcArgs aa;
      aa.K = K; aa.A_K = L->A_K; aa.ws = ws; aa.status = reinterpret_cast<int32_t *>(ws + lay.status);
      aa.seq_len = seq_len; aa.a_capacity = L->a_capacity; aa.sweep_base = lay.sweep; aa.sweep_stride = lay.sweep_stride;
      aa.sweeps = sweeps; aa.bsz = L->bsz; aa.q_heads = L->q_heads; aa.kv_heads = L->kv_heads; aa.head_dim = D; aa.r = R;
      aa.tol = tol;
      const int rc = launch_apply_tc(aa, stream);
      if (rc == LRQK_OK) pp.rows_elsewhere = 1;
      else if (rc != LRQK_EUNSUPPORTED) return rc;
    }
  }
  const unsigned apply_tiles = pp.rows_elsewhere ? 1u : (unsigned)ceil_div64(seq_len, kApplyRows);
  apply_kernel<T, R, D><<<dim3(apply_tiles, n_heads, 1), kFThreads, 0, stream>>>(pp);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

template <typename T, int D>
int dispatch_r(const lrqk_layer *L, const void *Q, const void *K, float *A_Q, float *A_K_init, int64_t seq_len,
               int sweeps, float tol, void *a_q_last, int32_t *sweeps_out, float *ws, cudaStream_t stream) {
  switch (L->r) {
    case 8: return run<T, 8, D>(L, Q, K, A_Q, A_K_init, seq_len, sweeps, tol, a_q_last, sweeps_out, ws, stream);
    case 16: return run<T, 16, D>(L, Q, K, A_Q, A_K_init, seq_len, sweeps, tol, a_q_last, sweeps_out, ws, stream);
    case 32: return run<T, 32, D>(L, Q, K, A_Q, A_K_init, seq_len, sweeps, tol, a_q_last, sweeps_out, ws, stream);
    case 64: return run<T, 64, D>(L, Q, K, A_Q, A_K_init, seq_len, sweeps, tol, a_q_last, sweeps_out, ws, stream);
    default: return LRQK_EUNSUPPORTED;
  }
}

// The d x r maps of the stopping sweep, copied out of the workspace: A_Q = Q X_Q, A_K = K X_K.
__global__ void factor_maps_kernel(const float *ws, FactorWs lay, int sweeps, const int32_t *sweeps_out, int dr,
                                   float *x_q_out, float *x_k_out) {
  const int n = blockIdx.x;
  int chosen = *sweeps_out - 1;
  if (chosen < 0) chosen = 0;
  if (chosen >= sweeps) chosen = sweeps - 1;
  const float *res = ws + lay.sweep + ((int64_t)n * sweeps + chosen) * lay.sweep_stride;  // X_Q, X_K, B_Q, B_K, ...
  for (int i = threadIdx.x; i < dr; i += blockDim.x) {
    if (x_q_out) x_q_out[(int64_t)n * dr + i] = res[i];
    if (x_k_out) x_k_out[(int64_t)n * dr + i] = res[dr + i];
  }
}

}  // namespace
}  // namespace lrqk

extern "C" int lrqk_prefill_factor_maps(const lrqk_layer *L, int64_t seq_len, int32_t sweeps, const int32_t *sweeps_out,
                                        const void *workspace, float *x_q_out, float *x_k_out, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!workspace || !sweeps_out || seq_len <= 0 || (!x_q_out && !x_k_out)) return LRQK_EINVAL;
  if (sweeps < 1) sweeps = 1;
  if (sweeps > kMaxSweeps) return LRQK_EUNSUPPORTED;
  const int n_heads = L->bsz * L->q_heads;
  const FactorWs lay = factor_ws_layout(n_heads, L->r, L->head_dim, sweeps, plan_gram_splits(n_heads, seq_len));
  factor_maps_kernel<<<n_heads, 256, 0, as_stream(stream)>>>(reinterpret_cast<const float *>(workspace), lay, sweeps,
                                                             sweeps_out, L->head_dim * L->r, x_q_out, x_k_out);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

extern "C" size_t lrqk_prefill_factorize_workspace_bytes(const lrqk_layer *L, int64_t seq_len) {
  using namespace lrqk;
  if (!L || seq_len <= 0) return 0;
  const int n_heads = L->bsz * L->q_heads;
  const FactorWs lay = factor_ws_layout(n_heads, L->r, L->head_dim, kMaxSweeps, plan_gram_splits(n_heads, seq_len));
  return (size_t)lay.total * sizeof(float);
}

extern "C" int lrqk_prefill_factorize(const lrqk_layer *L, const void *Q, const void *K, float *A_Q, float *A_K_init,
                                      int64_t seq_len, int32_t sweeps, float tol, void *a_q_last, int32_t *sweeps_out,
                                      void *workspace, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!Q || !K || !A_Q || !A_K_init || !a_q_last || !workspace || !L->A_K || !L->B_Q || !L->B_K) return LRQK_EINVAL;
  if (seq_len <= 0) return LRQK_EINVAL;
  if (seq_len > L->a_capacity) return LRQK_ECAPACITY;
  if (sweeps < 1) sweeps = 1;
  if (sweeps > kMaxSweeps) return LRQK_EUNSUPPORTED;
  if (ceil_div64(seq_len, kApplyRows) > 0x7FFFFFFF || L->bsz * L->q_heads > 65535) return LRQK_EUNSUPPORTED;
  float *ws = reinterpret_cast<float *>(workspace);
  cudaStream_t s = as_stream(stream);
  if (L->head_dim == 128) {
    LRQK_DISPATCH_DTYPE(L->dtype, T,
                        return (dispatch_r<T, 128>(L, Q, K, A_Q, A_K_init, seq_len, sweeps, tol, a_q_last, sweeps_out, ws, s)));
  } else if (L->head_dim == 64) {
    LRQK_DISPATCH_DTYPE(L->dtype, T,
                        return (dispatch_r<T, 64>(L, Q, K, A_Q, A_K_init, seq_len, sweeps, tol, a_q_last, sweeps_out, ws, s)));
  }
  return LRQK_EUNSUPPORTED;
}
