// Per-step rank-r projection of (q, k) and update of the right factors B_Q, B_K.
//
// Kernel 1 (project): one thread-block cluster per (batch, query head).
//   * CTA 0 is the solver.  While its peers stream, it loads B_Q and B_K, forms their r x r Gram
//     matrices and the vectors q B_Q^T, k B_K^T, q k^T, and solves for the initial k_hat.
//   * CTAs 1.. stream the active set (the k slot-table rows, then the m lite rows), cut into
//     equal shares: s_j = q . K_j from the resident keys, the matching rank-r rows a_j gathered
//     from A_K, and the partial sums  w = sum_j s_j a_j,  G = sum_j a_j^T a_j  in registers.
//     (A cluster of one CTA does both jobs in turn.)
//   * The partial sums meet in CTA 0 through distributed shared memory; it then runs the
//     alternating r x r solves and leaves every iterate in the workspace.
//   Each r x r system is a fixed symmetric positive definite matrix (a Gram matrix) plus a
//   rank-one term that changes from solve to solve.  The two fixed matrices are inverted once
//   (Gauss-Jordan without row exchanges, one warp, matrix rows in registers); every solve is
//   then a Sherman-Morrison update plus one step of iterative refinement, two small
//   matrix-vector products by one warp, instead of a fresh factorisation on the critical path.
//
// Kernel 2 (update): the early-exit test of the reference is a mean over ALL heads, so it can
// only be evaluated after kernel 1 has finished for every head.  Each CTA (one per head)
// re-derives the common stopping iteration from the per-head squared differences, picks that
// iterate, applies the line-searched rank-1 step to B_Q and B_K and writes q_hat and the new
// A_K row in the storage dtype.
#include <cooperative_groups.h>

#include "common.cuh"
#include "smallmat.cuh"

namespace cg = cooperative_groups;

namespace lrqk {
namespace {

constexpr int kPThreads = 256;
constexpr int kPWarps = kPThreads / 32;
constexpr int kBatch = 8;       // key rows a warp keeps in flight
constexpr int kGramPart = 4096; // floats of scratch for the per-group partial Gram matrices

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
  int32_t tile_rows;  // rows a streaming CTA handles per pass over its buffers
  float *ws;          // [N][max_iter][2R+2]
  // fused ring write (fuse_row >= 0): this kernel also stores the step's key/value into slot
  // fuse_row of the resident rows (and its position into lite_pos), which the ring-write kernel
  // does otherwise; the streaming CTAs take that row from k_new instead of from K_res
  const void *v_new;
  void *K_res_w, *V_res_w;
  int32_t *lite_pos_w;
  int32_t fuse_row, position;
};

// Rows of the streaming buffers (bounded so that the buffers stay near 40 KiB).
template <int R> constexpr int max_tile_rows() { return R >= 64 ? 160 : (R == 32 ? 320 : 512); }

// X^T X for a row-major X [nrows][ldx] with R columns, accumulated by all threads of the CTA.
// The R x R result is cut into 4 x 4 register tiles; the (R/4)^2 threads of a group cover it and
// the kPThreads / (R/4)^2 groups take every NG-th row each.  A thread loads its four row- and
// four column-operands with two 16-byte shared-memory loads per row of X.  The per-group
// partial sums are folded through `part` (kGramPart floats) into `out` (R x R, symmetric to the
// last bit because both triangles see the same operands in the same order).
template <int R>
__device__ __forceinline__ void gram_xtx(const float *X, int ldx, int nrows, float *part, float *out, bool add) {
  constexpr int TE = R / 4, TG = TE * TE, NG = kPThreads / TG;
  const int tid = threadIdx.x, grp = tid / TG, ty = (tid % TG) / TE, tx = tid % TE;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[a][c] = 0.0f;
#pragma unroll 4
  for (int row = grp; row < nrows; row += NG) {
    const float4 r4 = *reinterpret_cast<const float4 *>(X + row * ldx + 4 * ty);
    const float4 c4 = *reinterpret_cast<const float4 *>(X + row * ldx + 4 * tx);
    const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][c] = fmaf(rr[a], cc[c], acc[a][c]);
  }
  __syncthreads();  // `part` may still be in use by a previous call
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) part[grp * R * R + (4 * ty + a) * R + 4 * tx + c] = acc[a][c];
  __syncthreads();
  for (int i = tid; i < R * R; i += kPThreads) {
    float s = add ? out[i] : 0.0f;
#pragma unroll
    for (int g = 0; g < NG; ++g) s += part[g * R * R + i];
    out[i] = s;
  }
  __syncthreads();
}

// out[c] = sum_rows coef[row] * X[row][c] for a row-major X [nrows][ldx] with R columns.
template <int R>
__device__ __forceinline__ void weighted_colsum(const float *X, int ldx, int nrows, const float *coef, float *part,
                                                float *out, bool add) {
  constexpr int NGW = kPThreads / R;
  const int tid = threadIdx.x, c = tid % R, g = tid / R;
  float acc = 0.0f;
#pragma unroll 4
  for (int row = g; row < nrows; row += NGW) acc = fmaf(coef[row], X[row * ldx + c], acc);
  __syncthreads();
  part[g * R + c] = acc;
  __syncthreads();
  if (tid < R) {
    float s = add ? out[tid] : 0.0f;
#pragma unroll
    for (int gg = 0; gg < NGW; ++gg) s += part[gg * R + tid];
    out[tid] = s;
  }
  __syncthreads();
}

// x = (G + v^T v)^-1 b for symmetric G with a known inverse Gi (Sherman-Morrison), followed by one
// step of iterative refinement against G itself.  Executed by ONE warp; lane i owns row i (and
// i+32).  G and Gi are read column-wise (they are symmetric), which is free of bank conflicts.
// x and tmp are R floats of shared memory; x receives the result.
template <int R>
__device__ __forceinline__ void warp_rank1_solve(const float *G, const float *Gi, const float *v, const float *b,
                                                 float *x, float *tmp) {
  constexpr int RPL = (R + 31) / 32;
  const int lane = threadIdx.x & 31;
  float y[RPL], z[RPL], vi[RPL], bi[RPL], xv[RPL];
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    const int i = lane + 32 * t;
    y[t] = z[t] = 0.0f;
    vi[t] = i < R ? v[i] : 0.0f;
    bi[t] = i < R ? b[i] : 0.0f;
    if (i < R) {
#pragma unroll 8
      for (int j = 0; j < R; ++j) {
        const float gij = Gi[j * R + i];
        y[t] = fmaf(gij, b[j], y[t]);
        z[t] = fmaf(gij, v[j], z[t]);
      }
    }
  }
  float alpha = 0.0f, beta = 0.0f;
#pragma unroll
  for (int t = 0; t < RPL; ++t) { alpha = fmaf(vi[t], y[t], alpha); beta = fmaf(vi[t], z[t], beta); }
  alpha = warp_sum(alpha);
  beta = warp_sum(beta);
  const float inv = 1.0f / (1.0f + beta);
  float vx = 0.0f;
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    xv[t] = y[t] - z[t] * (alpha * inv);
    vx = fmaf(vi[t], xv[t], vx);
    if (lane + 32 * t < R) x[lane + 32 * t] = xv[t];
  }
  vx = warp_sum(vx);
  __syncwarp();
  // residual r = b - G x - v (v . x), then the same solve for the correction
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    const int i = lane + 32 * t;
    float r = bi[t] - vi[t] * vx;
    if (i < R) {
#pragma unroll 8
      for (int j = 0; j < R; ++j) r = fmaf(-G[j * R + i], x[j], r);
      tmp[i] = r;
    }
  }
  __syncwarp();
  float dalpha = 0.0f, dy[RPL];
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    const int i = lane + 32 * t;
    dy[t] = 0.0f;
    if (i < R) {
#pragma unroll 8
      for (int j = 0; j < R; ++j) dy[t] = fmaf(Gi[j * R + i], tmp[j], dy[t]);
    }
    dalpha = fmaf(vi[t], dy[t], dalpha);
  }
  dalpha = warp_sum(dalpha);
  __syncwarp();
#pragma unroll
  for (int t = 0; t < RPL; ++t)
    if (lane + 32 * t < R) x[lane + 32 * t] = xv[t] + dy[t] - z[t] * (dalpha * inv);
  __syncwarp();
}

template <typename T, int R, int D>
__global__ void __launch_bounds__(kPThreads, 2) project_kernel(ProjectParams p) {
  constexpr int EL = D / 32;       // key elements per lane
  constexpr int LDT = R + 4;       // leading dimension of the transposed right factors in shared memory

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int csize = (int)cluster.num_blocks();
  const int n = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b_idx = n / p.q_heads, h = n % p.q_heads;
  const int kvh = h / p.groups, kv_heads = p.q_heads / p.groups;
  const bool solver = rank == 0;
  const bool streamer = csize == 1 || rank > 0;
  const int n_streamers = csize == 1 ? 1 : csize - 1;

  extern __shared__ __align__(16) float sm[];
  float *Gp = sm;                         // [R][R] A^T A over this CTA's rows
  float *wp = Gp + R * R;                 // [R]    sum_j s_j a_j over this CTA's rows
  float *qs = wp + R;                     // [D]
  float *ks = qs + D;                     // [D]
  float *part = ks + D;                   // [kGramPart] partial sums of the group reductions
  float *region = part + kGramPart;
  // streaming buffers
  float *S = region;                                              // [tile_rows]
  int32_t *pos_s = reinterpret_cast<int32_t *>(S + p.tile_rows);  // [tile_rows]
  float *At = reinterpret_cast<float *>(pos_s + p.tile_rows);     // [tile_rows][R]
  // solver buffers: they share the region with the streaming buffers unless this CTA does both jobs
  float *sol = csize == 1 ? At + p.tile_rows * R : region;
  float *BtQ = sol;                       // [D][LDT] B_Q transposed
  float *BtK = BtQ + D * LDT;             // [D][LDT]
  float *GQ = BtK + D * LDT;              // [R][R]  B_Q B_Q^T (+ A^T A)
  float *GQi = GQ + R * R;
  float *GK = GQi + R * R;                // [R][R]  B_K B_K^T
  float *GKi = GK + R * R;
  float *vec = GKi + R * R;               // vectors of R: qrhs, kbk, khat, qhat, knew, rhs, tmp
  float *misc = vec + 7 * R;              // [4]
  float *qrhs = vec, *kbk = vec + R, *khat = vec + 2 * R, *qhat = vec + 3 * R, *knew = vec + 4 * R;
  float *rhs = vec + 5 * R, *tmpv = vec + 6 * R;

  pdl_launch_dependents();
  pdl_wait();
  const T *qg = reinterpret_cast<const T *>(p.q) + (int64_t)n * D;
  const T *kg = reinterpret_cast<const T *>(p.k_new) + ((int64_t)b_idx * kv_heads + kvh) * D;
  for (int e = tid; e < D; e += kPThreads) {
    qs[e] = Elt<T>::to_float(qg[e]);
    ks[e] = Elt<T>::to_float(kg[e]);
  }
  __syncthreads();

  // ---- streaming CTAs: their share of the active rows ------------------------------------------
  if (streamer) {
    const int n_act = p.k + p.m;
    const int srank = csize == 1 ? 0 : rank - 1;
    const int chunk = (n_act + n_streamers - 1) / n_streamers;
    const int j_begin = srank * chunk;
    const int j_end = min(n_act, j_begin + chunk);
    float qf[EL];
#pragma unroll
    for (int e = 0; e < EL; ++e) qf[e] = qs[lane * EL + e];
    const T *Kres = reinterpret_cast<const T *>(p.K_res) + (int64_t)n * n_act * D;
    const T *AK = reinterpret_cast<const T *>(p.A_K) + (int64_t)n * p.a_capacity * R;
    const int32_t *tab = p.table + (int64_t)n * p.k;
    bool first = true;
    for (int t0 = j_begin; t0 < j_end || first; t0 += p.tile_rows) {
      const int rows = max(0, min(p.tile_rows, j_end - t0));
      for (int i = tid; i < rows; i += kPThreads) {
        const int j = t0 + i;
        pos_s[i] = j == p.fuse_row ? p.position : (j < p.k ? tab[j] : p.lite_pos[j - p.k]);
      }
      __syncthreads();
      // rank-r rows of the tile's tokens: 16-byte pieces, gathered by all threads
      constexpr int CPR = R * (int)sizeof(T) / 16;  // 16-byte pieces per row
      constexpr int EPV = Elt<T>::kPerVec;
      for (int i = tid; i < rows * CPR; i += kPThreads) {
        const int row = i / CPR, c = i % CPR;
        float f[EPV];
        Elt<T>::unpack(ld16(AK + (int64_t)pos_s[row] * R + c * EPV), f);
#pragma unroll
        for (int e = 0; e < EPV; ++e) At[row * R + c * EPV + e] = f[e];
      }
      // s_j = q . K_j : a warp takes rows warp, warp + 8, ... with kBatch rows in flight
      for (int r0 = warp; r0 < rows; r0 += kPWarps * kBatch) {
        float kv[kBatch][EL];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int row = r0 + u * kPWarps;
          if (row < rows) RowLoad<T, EL>::run(Kres + (int64_t)(t0 + row) * D + lane * EL, kv[u]);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int row = r0 + u * kPWarps;
          float acc = 0.0f;
          if (row < rows) {
            // the step's own key is not in K_res yet when the ring write is fused (what was loaded for
            // that slot is the ring's previous occupant): take it from k_new
            const bool own = t0 + row == p.fuse_row;
#pragma unroll
            for (int e = 0; e < EL; ++e) acc = fmaf(own ? ks[lane * EL + e] : kv[u][e], qf[e], acc);
          }
          acc = warp_sum(acc);
          if (lane == 0 && row < rows) S[row] = acc;
        }
      }
      __syncthreads();
      gram_xtx<R>(At, R, rows, part, Gp, !first);
      weighted_colsum<R>(At, R, rows, S, part, wp, !first);
      first = false;
    }
  }

  // ---- solver CTA: everything that does not depend on the active rows ----------------------------
  if (solver && p.fuse_row >= 0) {  // fused ring write: 16-byte copies of the step's key and value
    constexpr int CH = D * (int)sizeof(T) / 16;
    const int64_t dst = ((int64_t)n * (p.k + p.m) + p.fuse_row) * D * (int64_t)sizeof(T);
    const int64_t src = ((int64_t)b_idx * kv_heads + kvh) * D * (int64_t)sizeof(T);
    if (tid < CH) st16(reinterpret_cast<char *>(p.K_res_w) + dst + tid * 16, ld16(reinterpret_cast<const char *>(p.k_new) + src + tid * 16));
    else if (tid < 2 * CH) st16(reinterpret_cast<char *>(p.V_res_w) + dst + (tid - CH) * 16,
                                ld16(reinterpret_cast<const char *>(p.v_new) + src + (tid - CH) * 16));
    if (n == 0 && tid == 2 * CH) p.lite_pos_w[p.fuse_row - p.k] = p.position;
  }
  if (solver) {
    const T *BQg = reinterpret_cast<const T *>(p.B_Q) + (int64_t)n * R * D;
    const T *BKg = reinterpret_cast<const T *>(p.B_K) + (int64_t)n * R * D;
    constexpr int EPV = Elt<T>::kPerVec;
    for (int i = tid; i < R * D / EPV; i += kPThreads) {
      const int a = (i * EPV) / D, e = (i * EPV) % D;
      float fq[EPV], fk[EPV];
      Elt<T>::unpack(ld16(BQg + (int64_t)i * EPV), fq);
      Elt<T>::unpack(ld16(BKg + (int64_t)i * EPV), fk);
#pragma unroll
      for (int x = 0; x < EPV; ++x) { BtQ[(e + x) * LDT + a] = fq[x]; BtK[(e + x) * LDT + a] = fk[x]; }
    }
    __syncthreads();
    gram_xtx<R>(BtQ, LDT, D, part, GQ, false);             // B_Q B_Q^T
    gram_xtx<R>(BtK, LDT, D, part, GK, false);             // B_K B_K^T
    weighted_colsum<R>(BtQ, LDT, D, qs, part, qrhs, false);  // q B_Q^T
    weighted_colsum<R>(BtK, LDT, D, ks, part, kbk, false);   // k B_K^T
    if (warp == 0) {
      float acc = 0.0f;
      for (int e = lane; e < D; e += 32) acc = fmaf(qs[e], ks[e], acc);
      acc = warp_sum(acc);
      if (lane == 0) misc[0] = acc;  // q k^T
    }
    __syncthreads();
    if (warp == 0) {  // invert B_K B_K^T, then k_hat0 = k B_K^T (B_K B_K^T)^-1
      warp_spd_inverse<R>(GK, GKi);
      for (int i = lane; i < R; i += 32) {
        float acc = 0.0f;
#pragma unroll 8
        for (int j = 0; j < R; ++j) acc = fmaf(GKi[j * R + i], kbk[j], acc);
        tmpv[i] = acc;
      }
      __syncwarp();
      // one refinement step against G_K itself
      for (int i = lane; i < R; i += 32) {
        float r = kbk[i];
#pragma unroll 8
        for (int j = 0; j < R; ++j) r = fmaf(-GK[j * R + i], tmpv[j], r);
        rhs[i] = r;
      }
      __syncwarp();
      for (int i = lane; i < R; i += 32) {
        float acc = tmpv[i];
#pragma unroll 8
        for (int j = 0; j < R; ++j) acc = fmaf(GKi[j * R + i], rhs[j], acc);
        khat[i] = acc;
      }
    }
  }

  cluster.sync();  // partial sums of every streaming CTA are in place
  if (!solver) {
    cluster.sync();  // stay resident until CTA 0 has read them
    return;
  }
  const int first_rank = csize == 1 ? 0 : 1;
  for (int i = tid; i < R * R / 4; i += kPThreads) {  // 16-byte remote loads, all peers in flight at once
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = first_rank; c < csize; ++c) {
      const float4 v = reinterpret_cast<const float4 *>(cluster.map_shared_rank(Gp, c))[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    float4 g = reinterpret_cast<float4 *>(GQ)[i];
    g.x += s.x; g.y += s.y; g.z += s.z; g.w += s.w;
    reinterpret_cast<float4 *>(GQ)[i] = g;  // B_Q B_Q^T + A^T A
  }
  if (tid < R) {
    float s = 0.0f;
    for (int c = first_rank; c < csize; ++c) s += cluster.map_shared_rank(wp, c)[tid];
    qrhs[tid] += s;  // q B_Q^T + (q K^T) A
  }
  cluster.sync();  // peers may retire

  float *ws = p.ws + (int64_t)n * p.max_iter * (2 * R + 2);
  if (warp == 0) {
    warp_spd_inverse<R>(GQ, GQi);
    const float qk = misc[0];
    for (int it = 0; it < p.max_iter; ++it) {
      // q_hat = (qrhs + qk * k_hat)(GQ + k_hat^T k_hat)^-1
      for (int i = lane; i < R; i += 32) rhs[i] = fmaf(qk, khat[i], qrhs[i]);
      __syncwarp();
      warp_rank1_solve<R>(GQ, GQi, khat, rhs, qhat, tmpv);
      // k_hat' = (kbk + qk * q_hat)(GK + q_hat^T q_hat)^-1
      for (int i = lane; i < R; i += 32) rhs[i] = fmaf(qk, qhat[i], kbk[i]);
      __syncwarp();
      warp_rank1_solve<R>(GK, GKi, qhat, rhs, knew, tmpv);
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
      }
      if (lane == 0) w[2 * R] = ssd;
      __syncwarp();
      for (int i = lane; i < R; i += 32) khat[i] = knew[i];
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
  int32_t *clear_word;  // optional: set to zero by the kernel
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
  pdl_launch_dependents();
  pdl_wait();

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
    if (n == 0 && p.clear_word) *p.clear_word = 0;
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

template <int R, int D>
size_t project_smem_bytes(int tile_rows, int csize) {
  const size_t common = (size_t)R * R + R + 2 * D + kGramPart;
  const size_t stream = (size_t)tile_rows * (2 + R);
  const size_t solve = 2 * (size_t)D * (R + 4) + 4 * (size_t)R * R + 7 * R + 4;
  return sizeof(float) * (common + (csize == 1 ? stream + solve : (stream > solve ? stream : solve)));
}

template <typename T, int R, int D>
int launch(const lrqk_layer *L, ProjectParams pp, const UpdateParams &up, cudaStream_t stream) {
  const int n_heads = L->bsz * L->q_heads;
  const int n_act = L->k + L->m;
  // CTAs per head: one solver plus streaming CTAs with at least ~128 rows each, while the grid stays
  // within about two CTAs per SM -- four when there are no more heads than SMs, where a short second
  // wave costs less than leaving a head's rows to one streaming CTA (measured: 128 heads 154 -> 134 us
  // with clusters of 4; 224 heads are quickest with one CTA per head, 78 us against 132 us with two)
  int csize = 1;
  const int cta_budget = n_heads <= kNumSMs ? 4 * kNumSMs : 2 * kNumSMs;
  while (csize < 8 && n_heads * csize * 2 <= cta_budget && n_act / (csize * 2 - 1) >= 128) csize *= 2;
  const int n_streamers = csize == 1 ? 1 : csize - 1;
  const int chunk = (n_act + n_streamers - 1) / n_streamers;
  const int passes = (chunk + max_tile_rows<R>() - 1) / max_tile_rows<R>();
  pp.tile_rows = ((chunk + passes - 1) / passes + 7) / 8 * 8;
  const size_t smem = project_smem_bytes<R, D>(pp.tile_rows, csize);
  auto kern = project_kernel<T, R, D>;
  static size_t smem_set = 0;
  if (smem > smem_set) {
    LRQK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    smem_set = smem;
  }
  LRQK_CUDA_TRY(launch_dependent(kern, dim3(csize, n_heads, 1), dim3(kPThreads), smem, stream, csize, pp));
  LRQK_CUDA_TRY(launch_dependent(update_kernel<T, R, D>, dim3(n_heads), dim3(D), 0, stream, 0, up));
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
  return lrqk::project_update_enqueue(L, q, k_new, max_iter, tol, append_row, q_hat, iters_out, workspace, nullptr,
                                      lrqk::as_stream(stream), nullptr, -1);
}

int lrqk::project_update_enqueue(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter, float tol,
                                 int64_t append_row, void *q_hat, int32_t *iters_out, void *workspace,
                                 int32_t *clear_word, cudaStream_t s, const void *v_new, int32_t lite_slot) {
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
  pp.tile_rows = 0;
  pp.ws = reinterpret_cast<float *>(workspace);
  pp.v_new = v_new; pp.K_res_w = L->K_res; pp.V_res_w = L->V_res; pp.lite_pos_w = L->lite_pos;
  pp.fuse_row = -1; pp.position = (int32_t)append_row;
  if (v_new) {
    if (lite_slot < 0 || lite_slot >= L->m || !L->V_res) return LRQK_EINVAL;
    pp.fuse_row = L->k + lite_slot;
  }
  UpdateParams up;
  up.A_K = L->A_K; up.B_Q = L->B_Q; up.B_K = L->B_K; up.q = q; up.k_new = k_new;
  up.ws = pp.ws; up.q_hat = q_hat; up.iters_out = iters_out;
  up.a_capacity = L->a_capacity; up.append_row = append_row;
  up.q_heads = L->q_heads; up.groups = pp.groups; up.max_iter = max_iter; up.n_heads = pp.n_heads;
  up.tol = tol;
  up.clear_word = clear_word;
  if (L->head_dim == 128) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, return (dispatch_r<T, 128>(L, pp, up, s)));
  } else if (L->head_dim == 64) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, return (dispatch_r<T, 64>(L, pp, up, s)));
  }
  return LRQK_EUNSUPPORTED;
}
