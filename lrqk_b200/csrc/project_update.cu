// Per-step rank-r projection of (q, k) and update of the right factors B_Q, B_K.
//
// Kernel 1 (project): one thread-block cluster per (batch, query head).  The active set -- the k
// slot-table rows followed by the m lite rows -- is cut over the CTAs of the cluster; each CTA
// streams its share of the resident keys once (s_j = q . K_j), gathers the matching rank-r rows
// of A_K and accumulates  w = sum_j s_j a_j  and  G = sum_j a_j^T a_j  in registers.  The
// partial sums meet in CTA 0 through distributed shared memory, which then runs the r x r
// solves (LU with partial pivoting, one warp, matrix in shared memory) for every alternation
// and leaves each iterate in the workspace.
//
// Kernel 2 (update): the early-exit test of the reference is a mean over ALL heads, so it can
// only be evaluated after kernel 1 has finished for every head.  Each CTA (one per head)
// re-derives the common stopping iteration from the per-head squared differences, picks that
// iterate, applies the line-searched rank-1 step to B_Q and B_K and writes q_hat and the new
// A_K row in the storage dtype.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace lrqk {
namespace {

constexpr int kPThreads = 256;
constexpr int kTileRows = 64;

template <typename T, int EL> struct RowLoad;
template <> struct RowLoad<float, 4> {
  __device__ static __forceinline__ void run(const float *p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4 *>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
};
template <> struct RowLoad<float, 2> {
  __device__ static __forceinline__ void run(const float *p, float (&f)[2]) {
    const float2 v = *reinterpret_cast<const float2 *>(p);
    f[0] = v.x; f[1] = v.y;
  }
};
template <> struct RowLoad<__nv_bfloat16, 4> {
  __device__ static __forceinline__ void run(const __nv_bfloat16 *p, float (&f)[4]) {
    const uint2 v = *reinterpret_cast<const uint2 *>(p);
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
  }
};
template <> struct RowLoad<__nv_bfloat16, 2> {
  __device__ static __forceinline__ void run(const __nv_bfloat16 *p, float (&f)[2]) {
    const uint32_t v = *reinterpret_cast<const uint32_t *>(p);
    f[0] = __uint_as_float(v << 16); f[1] = __uint_as_float(v & 0xFFFF0000u);
  }
};

struct ProjectParams {
  const void *A_K, *B_Q, *B_K, *K_res, *q, *k_new;
  const int32_t *table, *lite_pos;
  int64_t a_capacity;
  int32_t q_heads, groups, k, m, max_iter, n_heads;
  float *ws;  // [N][max_iter][2R+2]
};

// In-place solve of M x = b by LU with partial pivoting, executed by ONE warp.
// M: R x R, leading dimension LD (destroyed); b: R (overwritten with x).
template <int R, int LD>
__device__ void warp_lu_solve(float *M, float *b) {
  const int lane = threadIdx.x & 31;
  for (int c = 0; c < R; ++c) {
    float best = -1.0f;
    int bi = c;
    for (int i = lane; i < R; i += 32) {
      if (i >= c) {
        const float v = fabsf(M[i * LD + c]);
        if (v > best) { best = v; bi = i; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (bi != c) {
      for (int j = lane; j < R; j += 32) {
        const float t = M[c * LD + j];
        M[c * LD + j] = M[bi * LD + j];
        M[bi * LD + j] = t;
      }
      if (lane == 0) { const float t = b[c]; b[c] = b[bi]; b[bi] = t; }
    }
    __syncwarp();
    const float rp = 1.0f / M[c * LD + c];
    const float bc = b[c];
    for (int i = c + 1 + lane; i < R; i += 32) {
      const float l = M[i * LD + c] * rp;
      for (int j = c + 1; j < R; ++j) M[i * LD + j] = fmaf(-l, M[c * LD + j], M[i * LD + j]);
      b[i] = fmaf(-l, bc, b[i]);
    }
    __syncwarp();
  }
  for (int c = R - 1; c >= 0; --c) {
    const float xc = b[c] / M[c * LD + c];
    __syncwarp();
    if (lane == 0) b[c] = xc;
    for (int i = lane; i < c; i += 32) b[i] = fmaf(-M[i * LD + c], xc, b[i]);
    __syncwarp();
  }
}

template <typename T, int R, int D>
__global__ void __launch_bounds__(kPThreads) project_kernel(ProjectParams p) {
  constexpr int EL = D / 32;                   // key elements per lane
  constexpr int MT = R >= 16 ? R / 16 : 1;     // Gram micro-tile edge per thread
  constexpr int GT = R >= 16 ? 16 : R;         // threads per Gram edge
  constexpr int LDB = D + 1;                   // padded leading dimension of B in shared memory
  constexpr int LDM = R + 1;

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int csize = (int)cluster.num_blocks();
  const int n = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b_idx = n / p.q_heads, h = n % p.q_heads;
  const int kvh = h / p.groups, kv_heads = p.q_heads / p.groups;

  extern __shared__ __align__(16) float sm[];
  float *Gp = sm;                         // [R][R] partial Gram of this CTA
  float *wp = Gp + R * R;                 // [R]
  float *S = wp + R;                      // [kTileRows]
  float *At = S + kTileRows;              // [kTileRows][R]
  float *qs = At + kTileRows * R;         // [D]
  float *ks = qs + D;                     // [D]
  // rank 0 only:
  float *BQ = ks + D;                     // [R][LDB]
  float *BK = BQ + R * LDB;               // [R][LDB]
  float *GQ = BK + R * LDB;               // [R][R]   B_Q B_Q^T + A^T A
  float *GK = GQ + R * R;                 // [R][R]   B_K B_K^T
  float *Mw = GK + R * R;                 // [R][LDM] LU work matrix
  float *vec = Mw + R * LDM;              // 6 vectors of R: qrhs, kbk, khat, qhat, rhs, khat_new
  float *misc = vec + 6 * R;              // [4]

  const T *qg = reinterpret_cast<const T *>(p.q) + (int64_t)n * D;
  const T *kg = reinterpret_cast<const T *>(p.k_new) + ((int64_t)b_idx * kv_heads + kvh) * D;
  for (int e = tid; e < D; e += kPThreads) {
    qs[e] = Elt<T>::to_float(qg[e]);
    ks[e] = Elt<T>::to_float(kg[e]);
  }
  __syncthreads();

  // ---- phase 1: this CTA's share of the active rows -------------------------------------------
  const int n_act = p.k + p.m;
  const int chunk = (n_act + csize - 1) / csize;
  const int j_begin = rank * chunk;
  const int j_end = min(n_act, j_begin + chunk);

  float qf[EL];
#pragma unroll
  for (int e = 0; e < EL; ++e) qf[e] = qs[lane * EL + e];

  const T *Kres = reinterpret_cast<const T *>(p.K_res) + (int64_t)n * n_act * D;
  const T *AK = reinterpret_cast<const T *>(p.A_K) + (int64_t)n * p.a_capacity * R;
  const int32_t *tab = p.table + (int64_t)n * p.k;

  const int ty = tid / GT, tx = tid % GT;
  const bool gram_thread = tid < GT * GT;
  float gacc[MT][MT];
#pragma unroll
  for (int a = 0; a < MT; ++a)
#pragma unroll
    for (int c = 0; c < MT; ++c) gacc[a][c] = 0.0f;
  float wacc = 0.0f;

  for (int t0 = j_begin; t0 < j_end; t0 += kTileRows) {
    const int rows = min(kTileRows, j_end - t0);
    // (i) s_j = q . K_j : each warp takes rows warp, warp+8, ...; loads issued eight at a time
    constexpr int RPW = kTileRows / (kPThreads / 32);
    float kv[RPW][EL];
#pragma unroll
    for (int u = 0; u < RPW; ++u) {
      const int row = warp + u * (kPThreads / 32);
      if (row < rows) RowLoad<T, EL>::run(Kres + (int64_t)(t0 + row) * D + lane * EL, kv[u]);
      else {
#pragma unroll
        for (int e = 0; e < EL; ++e) kv[u][e] = 0.0f;
      }
    }
    // (ii) rank-r rows of the same tokens
#pragma unroll
    for (int u = 0; u < RPW; ++u) {
      const int row = warp + u * (kPThreads / 32);
      if (row < rows) {
        const int j = t0 + row;
        const int pos = j < p.k ? tab[j] : p.lite_pos[j - p.k];
        for (int c = lane; c < R; c += 32) At[row * R + c] = Elt<T>::to_float(AK[(int64_t)pos * R + c]);
      } else {
        for (int c = lane; c < R; c += 32) At[row * R + c] = 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < RPW; ++u) {
      const int row = warp + u * (kPThreads / 32);
      float acc = 0.0f;
#pragma unroll
      for (int e = 0; e < EL; ++e) acc = fmaf(kv[u][e], qf[e], acc);
      acc = warp_sum(acc);
      if (lane == 0) S[row] = row < rows ? acc : 0.0f;
    }
    __syncthreads();
    // (iii) accumulate w and G over the tile
    if (gram_thread) {
      for (int row = 0; row < rows; ++row) {
        float ar[MT], ac[MT];
#pragma unroll
        for (int a = 0; a < MT; ++a) { ar[a] = At[row * R + ty * MT + a]; ac[a] = At[row * R + tx * MT + a]; }
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
          for (int c = 0; c < MT; ++c) gacc[a][c] = fmaf(ar[a], ac[c], gacc[a][c]);
      }
    }
    if (tid < R) {
      for (int row = 0; row < rows; ++row) wacc = fmaf(S[row], At[row * R + tid], wacc);
    }
    __syncthreads();
  }
  if (gram_thread) {
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
      for (int c = 0; c < MT; ++c) Gp[(ty * MT + a) * R + tx * MT + c] = gacc[a][c];
  }
  if (tid < R) wp[tid] = wacc;

  cluster.sync();
  if (rank != 0) {
    cluster.sync();  // stay resident until CTA 0 has read the partial sums
    return;
  }

  // ---- phase 2 (CTA 0): combine, build the small systems, solve ---------------------------------
  for (int i = tid; i < R * R; i += kPThreads) {
    float s = Gp[i];
    for (int c = 1; c < csize; ++c) s += cluster.map_shared_rank(Gp, c)[i];
    GQ[i] = s;  // A^T A for now
  }
  if (tid < R) {
    float s = wp[tid];
    for (int c = 1; c < csize; ++c) s += cluster.map_shared_rank(wp, c)[tid];
    vec[tid] = s;  // (q K^T) A for now
  }
  cluster.sync();  // peers may retire

  const T *BQg = reinterpret_cast<const T *>(p.B_Q) + (int64_t)n * R * D;
  const T *BKg = reinterpret_cast<const T *>(p.B_K) + (int64_t)n * R * D;
  for (int i = tid; i < R * D; i += kPThreads) {
    const int a = i / D, e = i % D;
    BQ[a * LDB + e] = Elt<T>::to_float(BQg[i]);
    BK[a * LDB + e] = Elt<T>::to_float(BKg[i]);
  }
  __syncthreads();
  // Gram matrices of the right factors
  if (gram_thread) {
    float accq[MT][MT], acck[MT][MT];
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
      for (int c = 0; c < MT; ++c) { accq[a][c] = 0.0f; acck[a][c] = 0.0f; }
    for (int e = 0; e < D; ++e) {
      float rq[MT], cq[MT], rk[MT], ck[MT];
#pragma unroll
      for (int a = 0; a < MT; ++a) {
        rq[a] = BQ[(ty * MT + a) * LDB + e]; cq[a] = BQ[(tx * MT + a) * LDB + e];
        rk[a] = BK[(ty * MT + a) * LDB + e]; ck[a] = BK[(tx * MT + a) * LDB + e];
      }
#pragma unroll
      for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int c = 0; c < MT; ++c) {
          accq[a][c] = fmaf(rq[a], cq[c], accq[a][c]);
          acck[a][c] = fmaf(rk[a], ck[c], acck[a][c]);
        }
    }
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
      for (int c = 0; c < MT; ++c) {
        const int idx = (ty * MT + a) * R + tx * MT + c;
        GQ[idx] += accq[a][c];
        GK[idx] = acck[a][c];
      }
  }
  // q B_Q^T, k B_K^T (one warp per output, strided) and q k^T
  float *qrhs = vec, *kbk = vec + R, *khat = vec + 2 * R, *qhat = vec + 3 * R, *knew = vec + 5 * R;
  for (int a = warp; a < 2 * R + 1; a += kPThreads / 32) {
    float acc = 0.0f;
    if (a < R) {
      for (int e = lane; e < D; e += 32) acc = fmaf(qs[e], BQ[a * LDB + e], acc);
    } else if (a < 2 * R) {
      for (int e = lane; e < D; e += 32) acc = fmaf(ks[e], BK[(a - R) * LDB + e], acc);
    } else {
      for (int e = lane; e < D; e += 32) acc = fmaf(qs[e], ks[e], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      if (a < R) qrhs[a] += acc;       // q B_Q^T + (q K^T) A
      else if (a < 2 * R) kbk[a - R] = acc;
      else misc[0] = acc;
    }
  }
  __syncthreads();

  float *ws = p.ws + (int64_t)n * p.max_iter * (2 * R + 2);
  if (warp == 0) {
    const float qk = misc[0];
    // k_hat0 = k B_K^T (B_K B_K^T)^-1
    for (int i = lane; i < R * R; i += 32) Mw[(i / R) * LDM + (i % R)] = GK[i];
    for (int i = lane; i < R; i += 32) khat[i] = kbk[i];
    __syncwarp();
    warp_lu_solve<R, LDM>(Mw, khat);
    for (int it = 0; it < p.max_iter; ++it) {
      // q_hat = (qrhs + qk * k_hat)(GQ + k_hat^T k_hat)^-1
      for (int i = lane; i < R * R; i += 32) {
        const int a = i / R, c = i % R;
        Mw[a * LDM + c] = fmaf(khat[a], khat[c], GQ[i]);
      }
      for (int i = lane; i < R; i += 32) qhat[i] = fmaf(qk, khat[i], qrhs[i]);
      __syncwarp();
      warp_lu_solve<R, LDM>(Mw, qhat);
      // k_hat' = (kbk + qk * q_hat)(GK + q_hat^T q_hat)^-1
      for (int i = lane; i < R * R; i += 32) {
        const int a = i / R, c = i % R;
        Mw[a * LDM + c] = fmaf(qhat[a], qhat[c], GK[i]);
      }
      for (int i = lane; i < R; i += 32) knew[i] = fmaf(qk, qhat[i], kbk[i]);
      __syncwarp();
      warp_lu_solve<R, LDM>(Mw, knew);
      float ssd = 0.0f;
      for (int i = lane; i < R; i += 32) {
        const float dlt = khat[i] - knew[i];
        ssd = fmaf(dlt, dlt, ssd);
      }
      ssd = warp_sum(ssd);
      float *w = ws + (int64_t)it * (2 * R + 2);
      for (int i = lane; i < R; i += 32) {
        w[i] = qhat[i];
        w[R + i] = knew[i];
        khat[i] = knew[i];
      }
      if (lane == 0) w[2 * R] = ssd;
      __syncwarp();
    }
  }
}

struct UpdateParams {
  void *A_K, *B_Q, *B_K;
  const void *q, *k_new;
  const float *ws;
  void *q_hat;
  int32_t *iters_out;
  int64_t a_capacity, append_row;
  int32_t q_heads, groups, max_iter, n_heads;
  float tol;
};

template <typename T, int R, int D>
__global__ void __launch_bounds__(D) update_kernel(UpdateParams p) {
  const int n = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b_idx = n / p.q_heads, h = n % p.q_heads;
  const int kvh = h / p.groups, kv_heads = p.q_heads / p.groups;
  constexpr int W = 2 * R + 2;
  __shared__ float delta[8];
  __shared__ float hat[2][R];
  __shared__ float red[2][4][D / 32];
  __shared__ int chosen;

  // common stopping iteration: mean over all heads of the squared change of k_hat
  for (int it = warp; it < p.max_iter && it < 8; it += D / 32) {
    float s = 0.0f;
    for (int hh = lane; hh < p.n_heads; hh += 32) s += p.ws[((int64_t)hh * p.max_iter + it) * W + 2 * R];
    s = warp_sum(s);
    if (lane == 0) delta[it] = s / (float)(p.n_heads * R);
  }
  __syncthreads();
  if (tid == 0) {
    int c = p.max_iter - 1;
    for (int it = 0; it < p.max_iter; ++it) {
      if (delta[it] < p.tol) { c = it; break; }
    }
    chosen = c;
    if (n == 0 && p.iters_out) *p.iters_out = c + 1;
  }
  __syncthreads();
  const float *w = p.ws + ((int64_t)n * p.max_iter + chosen) * W;
  if (tid < R) { hat[0][tid] = w[tid]; hat[1][tid] = w[R + tid]; }
  __syncthreads();

  T *Bg[2] = {reinterpret_cast<T *>(p.B_Q) + (int64_t)n * R * D, reinterpret_cast<T *>(p.B_K) + (int64_t)n * R * D};
  const T *xg[2] = {reinterpret_cast<const T *>(p.q) + (int64_t)n * D,
                    reinterpret_cast<const T *>(p.k_new) + ((int64_t)b_idx * kv_heads + kvh) * D};
  // thread e owns column e of both right factors
  const int e = tid;
  float col[2][R], t[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    float acc = 0.0f;
#pragma unroll
    for (int a = 0; a < R; ++a) {
      col[s][a] = Elt<T>::to_float(Bg[s][a * D + e]);
      acc = fmaf(hat[s][a], col[s][a], acc);
    }
    t[s] = acc - Elt<T>::to_float(xg[s][e]);  // (x_hat B - x)[e]
  }
  // |dB|^2 = sum_{a,e} (x_hat[a] t[e])^2 ;  |x_hat dB|^2 = sum_e (sum_a x_hat[a]^2 t[e])^2
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    float n2 = 0.0f, h2 = 0.0f;
#pragma unroll
    for (int a = 0; a < R; ++a) {
      const float dBae = hat[s][a] * t[s];
      n2 = fmaf(dBae, dBae, n2);
      h2 = fmaf(hat[s][a], dBae, h2);
    }
    n2 = warp_sum(n2);
    float hh = warp_sum(h2 * h2);
    if (lane == 0) { red[s][0][warp] = n2; red[s][1][warp] = hh; }
  }
  __syncthreads();
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    float n2 = 0.0f, hh = 0.0f;
#pragma unroll
    for (int wv = 0; wv < D / 32; ++wv) { n2 += red[s][0][wv]; hh += red[s][1][wv]; }
    const float eta = n2 / (hh + 1e-6f);
#pragma unroll
    for (int a = 0; a < R; ++a) {
      const float dBae = hat[s][a] * t[s];
      Bg[s][a * D + e] = Elt<T>::from_float(col[s][a] - eta * dBae);
    }
  }
  if (tid < R) {
    reinterpret_cast<T *>(p.q_hat)[(int64_t)n * R + tid] = Elt<T>::from_float(hat[0][tid]);
    reinterpret_cast<T *>(p.A_K)[((int64_t)n * p.a_capacity + p.append_row) * R + tid] = Elt<T>::from_float(hat[1][tid]);
  }
}

template <typename T, int R, int D>
size_t project_smem_bytes() {
  return sizeof(float) * (size_t)(R * R + R + kTileRows + kTileRows * R + 2 * D + 2 * R * (D + 1) + 2 * R * R +
                                  R * (R + 1) + 6 * R + 4);
}

template <typename T, int R, int D>
int launch(const lrqk_layer *L, const ProjectParams &pp, const UpdateParams &up, cudaStream_t stream) {
  const int n_heads = L->bsz * L->q_heads;
  const size_t smem = project_smem_bytes<T, R, D>();
  auto kern = project_kernel<T, R, D>;
  static bool attr_set = false;
  if (!attr_set) {
    LRQK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set = true;
  }
  // CTAs per head: as many as keep the grid within about two CTAs per SM, at least 64 rows each
  int csize = 1;
  while (csize < 8 && n_heads * csize * 2 <= 2 * kNumSMs && (L->k + L->m) / (csize * 2) >= kTileRows) csize *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(csize, n_heads, 1);
  cfg.blockDim = dim3(kPThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  LRQK_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, pp));
  update_kernel<T, R, D><<<n_heads, D, 0, stream>>>(up);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

template <typename T, int D>
int dispatch_r(const lrqk_layer *L, const ProjectParams &pp, const UpdateParams &up, cudaStream_t stream) {
  switch (L->r) {
    case 8: return launch<T, 8, D>(L, pp, up, stream);
    case 16: return launch<T, 16, D>(L, pp, up, stream);
    case 32: return launch<T, 32, D>(L, pp, up, stream);
    case 64: return launch<T, 64, D>(L, pp, up, stream);
    default: return LRQK_EUNSUPPORTED;
  }
}

}  // namespace
}  // namespace lrqk

extern "C" size_t lrqk_decode_project_update_workspace_bytes(const lrqk_layer *L, int32_t max_iter) {
  if (!L || max_iter < 0) return 0;
  const int it = max_iter < 1 ? 1 : max_iter;
  return sizeof(float) * (size_t)L->bsz * L->q_heads * it * (2 * L->r + 2);
}

extern "C" int lrqk_decode_project_update(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter,
                                          float tol, int64_t append_row, void *q_hat, int32_t *iters_out,
                                          void *workspace, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!q || !k_new || !q_hat || !workspace) return LRQK_EINVAL;
  if (!L->A_K || !L->B_Q || !L->B_K || !L->K_res || !L->table || !L->lite_pos) return LRQK_EINVAL;
  if (append_row < 0 || append_row >= L->a_capacity) return LRQK_ECAPACITY;
  if (max_iter < 1) max_iter = 1;  // the reference runs at least one alternation
  if (max_iter > 8) return LRQK_EUNSUPPORTED;
  ProjectParams pp;
  pp.A_K = L->A_K; pp.B_Q = L->B_Q; pp.B_K = L->B_K; pp.K_res = L->K_res; pp.q = q; pp.k_new = k_new;
  pp.table = L->table; pp.lite_pos = L->lite_pos;
  pp.a_capacity = L->a_capacity;
  pp.q_heads = L->q_heads; pp.groups = L->q_heads / L->kv_heads; pp.k = L->k; pp.m = L->m;
  pp.max_iter = max_iter; pp.n_heads = L->bsz * L->q_heads;
  pp.ws = reinterpret_cast<float *>(workspace);
  UpdateParams up;
  up.A_K = L->A_K; up.B_Q = L->B_Q; up.B_K = L->B_K; up.q = q; up.k_new = k_new;
  up.ws = pp.ws; up.q_hat = q_hat; up.iters_out = iters_out;
  up.a_capacity = L->a_capacity; up.append_row = append_row;
  up.q_heads = L->q_heads; up.groups = pp.groups; up.max_iter = max_iter; up.n_heads = pp.n_heads;
  up.tol = tol;
  cudaStream_t s = as_stream(stream);
  if (L->head_dim == 128) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, return (dispatch_r<T, 128>(L, pp, up, s)));
  } else if (L->head_dim == 64) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, return (dispatch_r<T, 64>(L, pp, up, s)));
  }
  return LRQK_EUNSUPPORTED;
}
