// Per-step rank-r projection of (q, k) and update of the right factors B_Q, B_K.
//
// Kernel 1 (project): one thread-block cluster per (batch, query head).
//   * CTA 0 is the solver.  While its peers stream, it loads B_Q and B_K (row-major, fp32, in
//     shared memory), forms their r x r Gram matrices and the vectors q B_Q^T, k B_K^T, q k^T,
//     inverts B_K B_K^T and solves for the initial k_hat.
//   * CTAs 1.. stream the active set (the k slot-table rows, then the m lite rows), cut into equal
//     shares.  A share's resident keys travel through a ring of shared-memory stages filled by
//     bulk asynchronous copies (cp.async.bulk completing on mbarriers; every stage of the ring is
//     requested before the first is waited for), the matching rank-r rows a_j are gathered from
//     A_K a few stages ahead into registers.  Per stage: s_j = q . K_j, then the partial sums
//     w = sum_j s_j a_j and G = sum_j a_j^T a_j are accumulated in registers (4 x 4 tiles of G per
//     thread) -- they leave the registers once, when the share is done.
//     (A cluster of one CTA does both jobs in turn, the copies of its first stages in flight
//     while it prepares the solver side.)
//   * Each streaming CTA stores its partial sums into its own slot of the SOLVER's shared memory
//     (distributed shared memory, plain remote stores); one cluster barrier later CTA 0 adds the
//     slots in rank order and runs the alternating r x r solves, leaving every iterate in the
//     workspace.
//   Each r x r system is a fixed symmetric positive definite matrix (a Gram matrix) plus a
//   rank-one term that changes from solve to solve.  The two fixed matrices are inverted once, by
//   a blocked Gauss-Jordan elimination without row exchanges in which every thread owns one 4 x 4
//   tile (r/4 steps of two barriers each; the 4 x 4 pivot block is inverted in closed form through
//   its 2 x 2 Schur complement).  Every solve is then a Sherman-Morrison update plus one step of
//   iterative refinement -- matrix-vector products by one warp with four independent partial sums
//   per row -- instead of a fresh factorisation on the critical path.
//
// Kernel 2 (update): the early-exit test of the reference is a mean over ALL heads, so it can
// only be evaluated after kernel 1 has finished for every head.  Each CTA (one per head)
// re-derives the common stopping iteration from the per-head squared differences, picks that
// iterate, applies the line-searched rank-1 step to B_Q and B_K and writes q_hat and the new
// A_K row in the storage dtype.
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"
#include "smallmat.cuh"
#include "tc_common.cuh"
#include "update_head.cuh"

namespace cg = cooperative_groups;

namespace lrqk {
namespace {

constexpr int kPThreads = 256;
constexpr int kPWarps = kPThreads / 32;
constexpr int kStageBytesK = 16 * 1024;  // resident keys per ring stage
constexpr int kRing = 4;                 // stages of the key ring
constexpr int kAhead = 4;                // stages the gather of the rank-r rows runs ahead of their use

struct ProjectParams {
  const void *A_K, *B_Q, *B_K, *K_res, *q, *k_new;
  const int32_t *table, *lite_pos;
  int64_t a_capacity;
  int32_t q_heads, groups, k, m, max_iter, n_heads;
  float lam_own, lam_act;  // weights of the new token's own q k^T term and of the active set's terms (:462-495)
  float *ws;          // [N][max_iter][2R+2]
  int32_t *status;    // set to LRQK_ETIMEOUT if a bounded wait ran out
  int32_t *clear_word;  // optional: set to zero by head 0's solver CTA at its end (the fused step's miss-list length)
  // fused ring write (fuse_row >= 0): this kernel also stores the step's key/value into slot
  // fuse_row of the resident rows (and its position into lite_pos), which the ring-write kernel
  // does otherwise; the streaming CTAs take that row from k_new instead of from K_res
  const void *v_new;
  void *K_res_w, *V_res_w;
  int32_t *lite_pos_w;
  int32_t fuse_row, position;
};

// ---- shared-memory plan ---------------------------------------------------------------------------
// Dynamic shared memory of a CTA, in this order (sizes in floats unless noted):
//   [operand tiles of the tensor-core Gram: bf16 only, 3 x 8 KiB, 1024-byte aligned]
//   [common: q, k, mbarriers, the partial-sum slots (solver CTA only)]
//   [streaming buffers]   [solver buffers]
// In a cluster the streaming CTAs have no solver buffers and the solver CTA has no streaming buffers
// (the two regions overlap); a cluster of one CTA has both.
constexpr int kTileBytes = 64 * 128;  // one operand tile: 64 rows (the contraction index) of 64 bf16 columns

template <typename T, int R, int D>
struct Plan {
  static constexpr bool TC = sizeof(T) == 2;            // bf16: the r x r Grams run on the tensor cores
  static constexpr int RB = D * (int)sizeof(T);         // bytes of a key row
  static constexpr int SR = kStageBytesK / RB > 64 ? 64 : kStageBytesK / RB;  // rows per stage (an operand tile holds 64)
  static constexpr int LDB = D + 4;                     // leading dimension of the right factors (fp32 path)
  static constexpr int LDG = R + 4;                     // leading dimension of the r x r matrices
  static constexpr int SLOT = R * R + R;                // one streaming CTA's partial sums: G then w
  static constexpr int tile_bytes = TC ? 3 * kTileBytes : 0;
  // common
  static constexpr int o_qs = 0;
  static constexpr int o_ks = o_qs + D;
  static constexpr int o_bars = o_ks + D;               // kRing + 4 mbarriers (2 floats each)
  static constexpr int o_slots = o_bars + 2 * (kRing + 4) + 4;
  __host__ __device__ static constexpr int common_floats(int n_slots) { return (o_slots + n_slots * SLOT + 31) / 32 * 32; }
  // streaming region
  static constexpr int s_ring = 0;                                   // kRing * kStageBytesK bytes
  static constexpr int s_At = s_ring + kRing * kStageBytesK / 4;     // [2][SR][R] fp32 (fp32 path only)
  static constexpr int s_S = s_At + (TC ? 0 : 2 * SR * R);           // [2][SR]
  static constexpr int s_pos = s_S + 2 * SR;                         // [rows of the share] int32
  __host__ __device__ static constexpr int stream_floats(int share_rows) { return (s_pos + share_rows + 31) / 32 * 32; }
  // solver region
  static constexpr int v_BQ = 0;                                     // [R][LDB]  (fp32 path only)
  static constexpr int v_BK = v_BQ + (TC ? 0 : R * LDB);
  static constexpr int v_GQ = v_BK + (TC ? 0 : R * LDB);             // [R][LDG]  B_Q B_Q^T (+ A^T A)
  static constexpr int v_GQi = v_GQ + R * LDG;
  static constexpr int v_GK = v_GQi + R * LDG;
  static constexpr int v_GKi = v_GK + R * LDG;
  static constexpr int v_vec = v_GKi + R * LDG;                      // 8 vectors of R
  static constexpr int v_misc = v_vec + 8 * R;
  static constexpr int v_part = v_misc + 4;                          // partial Grams of the thread groups (fp32 path)
  static constexpr int solver_floats =
      v_part + ((TC || R >= 64) ? 0 : (kPThreads / ((R / 4) * (R / 4))) * R * R);
  // (the streaming CTAs of the fp32 path fold their thread groups through the key ring once the streaming is over)
};

// ---- small helpers ----------------------------------------------------------------------------------
template <typename T> struct Piece;  // a 16-byte piece of a row as floats
template <> struct Piece<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[4]) { Elt<float>::unpack(v, f); }
};
template <> struct Piece<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[8]) { Elt<__nv_bfloat16>::unpack(v, f); }
};

// dot of a row-major fp32 matrix row with a vector, four independent partial sums (short dependency chains)
template <int R>
__device__ __forceinline__ float col_dot4(const float *M, int ld, int i, const float *x) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
  for (int j = 0; j < R; j += 4) {
    a0 = fmaf(M[(j + 0) * ld + i], x[j + 0], a0);
    a1 = fmaf(M[(j + 1) * ld + i], x[j + 1], a1);
    a2 = fmaf(M[(j + 2) * ld + i], x[j + 2], a2);
    a3 = fmaf(M[(j + 3) * ld + i], x[j + 3], a3);
  }
  return (a0 + a1) + (a2 + a3);
}

// Inverse of a symmetric positive definite 4 x 4 block through the Schur complement of its leading
// 2 x 2 block (two reciprocals on the dependency chain).
__device__ __forceinline__ void spd4_inverse(const float (&a)[4][4], float (&x)[4][4]) {
  // P = A11^-1
  const float d1 = fast_rcp(a[0][0] * a[1][1] - a[0][1] * a[1][0]);
  const float p00 = a[1][1] * d1, p01 = -a[0][1] * d1, p10 = -a[1][0] * d1, p11 = a[0][0] * d1;
  // U = P A12 (2x2), S = A22 - A21 U
  const float u00 = p00 * a[0][2] + p01 * a[1][2], u01 = p00 * a[0][3] + p01 * a[1][3];
  const float u10 = p10 * a[0][2] + p11 * a[1][2], u11 = p10 * a[0][3] + p11 * a[1][3];
  const float s00 = a[2][2] - (a[2][0] * u00 + a[2][1] * u10), s01 = a[2][3] - (a[2][0] * u01 + a[2][1] * u11);
  const float s10 = a[3][2] - (a[3][0] * u00 + a[3][1] * u10), s11 = a[3][3] - (a[3][0] * u01 + a[3][1] * u11);
  const float d2 = fast_rcp(s00 * s11 - s01 * s10);
  const float t00 = s11 * d2, t01 = -s01 * d2, t10 = -s10 * d2, t11 = s00 * d2;  // T = S^-1
  // V = A21 P (2x2);  X22 = T, X12 = -U T, X21 = -T V, X11 = P + U T V
  const float v00 = a[2][0] * p00 + a[2][1] * p10, v01 = a[2][0] * p01 + a[2][1] * p11;
  const float v10 = a[3][0] * p00 + a[3][1] * p10, v11 = a[3][0] * p01 + a[3][1] * p11;
  const float w00 = t00 * v00 + t01 * v10, w01 = t00 * v01 + t01 * v11;  // W = T V
  const float w10 = t10 * v00 + t11 * v10, w11 = t10 * v01 + t11 * v11;
  x[2][2] = t00; x[2][3] = t01; x[3][2] = t10; x[3][3] = t11;
  x[2][0] = -w00; x[2][1] = -w01; x[3][0] = -w10; x[3][1] = -w11;
  x[0][2] = -(u00 * t00 + u01 * t10); x[0][3] = -(u00 * t01 + u01 * t11);
  x[1][2] = -(u10 * t00 + u11 * t10); x[1][3] = -(u10 * t01 + u11 * t11);
  x[0][0] = p00 + u00 * w00 + u01 * w10; x[0][1] = p01 + u00 * w01 + u01 * w11;
  x[1][0] = p10 + u10 * w00 + u11 * w10; x[1][1] = p11 + u10 * w01 + u11 * w11;
}

// In-place inverse of the symmetric positive definite R x R matrix W (leading dimension ld, shared
// memory) by blocked Gauss-Jordan elimination without row exchanges.  All kPThreads threads call;
// thread t < (R/4)^2 owns the 4 x 4 tile (t / (R/4), t % (R/4)).  A step reads the pivot block, the
// tile's part of the pivot block column and of the pivot block row, then, behind a barrier, every
// owner writes its tile back: two barriers per step, R/4 steps.
template <int R>
__device__ __forceinline__ void cta_spd_inverse(float *W, int ld) {
  constexpr int NB = R / 4;
  const int tid = threadIdx.x;
  const bool owner = tid < NB * NB;
  const int bi = owner ? tid / NB : 0, bj = owner ? tid % NB : 0;
  float t[4][4];
  if (owner) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = *reinterpret_cast<const float4 *>(W + (4 * bi + i) * ld + 4 * bj);
      t[i][0] = v.x; t[i][1] = v.y; t[i][2] = v.z; t[i][3] = v.w;
    }
  }
#pragma unroll 1
  for (int p = 0; p < NB; ++p) {
    if (owner) {
      float piv[4][4], f[4][4], rw[4][4], dinv[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 a = *reinterpret_cast<const float4 *>(W + (4 * p + i) * ld + 4 * p);
        const float4 b = *reinterpret_cast<const float4 *>(W + (4 * bi + i) * ld + 4 * p);
        const float4 c = *reinterpret_cast<const float4 *>(W + (4 * p + i) * ld + 4 * bj);
        piv[i][0] = a.x; piv[i][1] = a.y; piv[i][2] = a.z; piv[i][3] = a.w;
        f[i][0] = b.x; f[i][1] = b.y; f[i][2] = b.z; f[i][3] = b.w;
        rw[i][0] = c.x; rw[i][1] = c.y; rw[i][2] = c.z; rw[i][3] = c.w;
      }
      spd4_inverse(piv, dinv);
      if (bi == p && bj == p) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) t[i][j] = dinv[i][j];
      } else if (bj == p) {  // pivot block column: -F Dinv
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float s = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) s = fmaf(f[i][c], dinv[c][j], s);
            t[i][j] = -s;
          }
      } else {
        float rn[4][4];  // Dinv * (pivot block row)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float s = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) s = fmaf(dinv[i][c], rw[c][j], s);
            rn[i][j] = s;
          }
        if (bi == p) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) t[i][j] = rn[i][j];
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float s = t[i][j];
#pragma unroll
              for (int c = 0; c < 4; ++c) s = fmaf(-f[i][c], rn[c][j], s);
              t[i][j] = s;
            }
        }
      }
    }
    __syncthreads();  // every owner has read the old pivot row and column
    if (owner) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4 *>(W + (4 * bi + i) * ld + 4 * bj) = make_float4(t[i][0], t[i][1], t[i][2], t[i][3]);
    }
    __syncthreads();
  }
}

// x = (G + lam v^T v)^-1 b for symmetric G with a known inverse Gi (Sherman-Morrison), followed by one
// step of iterative refinement against G itself.  (lam = 1 leaves every product below exact.)  Executed by ONE warp; lane i owns row i (and
// i+32).  G and Gi are read column-wise (they are symmetric), which is free of bank conflicts.
// x and tmp are R floats of shared memory; x receives the result.
template <int R>
__device__ __forceinline__ void warp_rank1_solve(const float *G, const float *Gi, int ld, const float *v, float lam,
                                                 const float *b, float *x, float *tmp) {
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
      y[t] = col_dot4<R>(Gi, ld, i, b);
      z[t] = col_dot4<R>(Gi, ld, i, v);
    }
  }
  float alpha = 0.0f, beta = 0.0f;
#pragma unroll
  for (int t = 0; t < RPL; ++t) { alpha = fmaf(vi[t], y[t], alpha); beta = fmaf(vi[t], z[t], beta); }
  alpha = warp_sum(alpha);
  beta = warp_sum(beta);
  const float inv = lam / (1.0f + lam * beta);
  float vx = 0.0f;
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    xv[t] = y[t] - z[t] * (alpha * inv);
    vx = fmaf(vi[t], xv[t], vx);
    if (lane + 32 * t < R) x[lane + 32 * t] = xv[t];
  }
  vx = warp_sum(vx);
  __syncwarp();
  // residual r = b - G x - lam v (v . x), then the same solve for the correction
  vx *= lam;
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    const int i = lane + 32 * t;
    if (i < R) tmp[i] = bi[t] - vi[t] * vx - col_dot4<R>(G, ld, i, x);
  }
  __syncwarp();
  float dalpha = 0.0f, dy[RPL];
#pragma unroll
  for (int t = 0; t < RPL; ++t) {
    const int i = lane + 32 * t;
    dy[t] = i < R ? col_dot4<R>(Gi, ld, i, tmp) : 0.0f;
    dalpha = fmaf(vi[t], dy[t], dalpha);
  }
  dalpha = warp_sum(dalpha);
  __syncwarp();
#pragma unroll
  for (int t = 0; t < RPL; ++t)
    if (lane + 32 * t < R) x[lane + 32 * t] = xv[t] + dy[t] - z[t] * (dalpha * inv);
  __syncwarp();
}

// B B^T for a row-major B [R][ld] with D columns (fp32, shared memory) into G [R][ldg].  The R x R
// result is cut into 4 x 4 register tiles with STRIDED rows and columns (tile (ty, tx) holds rows
// ty + i R/4 and columns tx + j R/4, so that the lanes of a warp read neighbouring rows of B, which
// sit four banks apart); the 256 / (R/4)^2 thread groups split the D columns of B and their partial
// tiles are added in group order through `part` ((groups) x R x R floats).
template <int R, int D>
__device__ __forceinline__ void gram_bbt(const float *B, int ld, float *part, float *G, int ldg) {
  constexpr int TE = R / 4, TG = TE * TE, NG = kPThreads / TG;
  constexpr int DG = D / NG;  // columns per group (a multiple of 4 for every supported shape, or D itself)
  const int tid = threadIdx.x, grp = tid / TG, ty = (tid % TG) / TE, tx = tid % TE;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[a][c] = 0.0f;
  if constexpr (DG >= 4) {
#pragma unroll 2
    for (int e = grp * DG; e < (grp + 1) * DG; e += 4) {
      float4 rr[4], cc[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        rr[a] = *reinterpret_cast<const float4 *>(B + (ty + a * TE) * ld + e);
        cc[a] = *reinterpret_cast<const float4 *>(B + (tx + a * TE) * ld + e);
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          acc[a][c] = fmaf(rr[a].x, cc[c].x, acc[a][c]);
          acc[a][c] = fmaf(rr[a].y, cc[c].y, acc[a][c]);
          acc[a][c] = fmaf(rr[a].z, cc[c].z, acc[a][c]);
          acc[a][c] = fmaf(rr[a].w, cc[c].w, acc[a][c]);
        }
    }
  } else {
    for (int e = grp * DG; e < (grp + 1) * DG; ++e) {
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][c] = fmaf(B[(ty + a * TE) * ld + e], B[(tx + c * TE) * ld + e], acc[a][c]);
    }
  }
  if constexpr (NG == 1) {
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) G[(ty + a * TE) * ldg + tx + c * TE] = acc[a][c];
    __syncthreads();
  } else {
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) part[grp * R * R + (ty + a * TE) * R + tx + c * TE] = acc[a][c];
    __syncthreads();
    for (int i = tid; i < R * R; i += kPThreads) {
      float s = 0.0f;
#pragma unroll
      for (int g = 0; g < NG; ++g) s += part[g * R * R + i];
      G[(i / R) * ldg + i % R] = s;
    }
    __syncthreads();
  }
}

// Address of the 16-byte chunk `chunk` of row `row` inside an operand tile (128-byte swizzle: the chunk
// index is XORed with the row index modulo 8).
__device__ __forceinline__ uint32_t tile_chunk(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// X^T X of one operand tile X [64 rows][64 bf16 columns] accumulated into the TMEM columns at `acc`
// (lanes 0..63 = the first index, columns 0..63 = the second): four tcgen05 MMAs of 16 rows each, issued
// by ONE thread.  The instruction is M128 N64; the upper 64 rows of its left operand read the all-zero
// tile `zero` (so lanes 64..127 of the accumulator stay zero).
__device__ __forceinline__ void gram_tile_mma(uint32_t tile, uint32_t zero, uint32_t acc, bool accumulate_first) {
  constexpr uint32_t kIdesc = tc::umma_idesc_bf16_mn(128, 64);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    const uint32_t off = ks * 2048;  // 16 rows of 128 bytes
    tc::umma_bf16(acc, tc::umma_desc_mn_sw128(tile + off, zero - tile, 1024), tc::umma_desc_mn_sw128(tile + off, kTileBytes, 1024),
                  kIdesc, (accumulate_first || ks > 0) ? 1u : 0u);
  }
}

// The R x R accumulator at TMEM column `col` into shared memory `dst` (row-major, leading dimension ld),
// or straight into another CTA's shared memory: warps 0 and 1 (TMEM lanes 0..63), lane = row.
template <int R>
__device__ __forceinline__ void gram_from_tmem(uint32_t tmem_base, uint32_t col, float *dst, int ld) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < 2 && warp * 32 < R) {  // warp-uniform
    const int row = warp * 32 + lane;
    uint32_t v[32];
#pragma unroll
    for (int c0 = 0; c0 < R; c0 += 32) {
      tc::tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + col + c0, v);
      if (row < R) {
#pragma unroll
        for (int j = 0; j < 32 && j < R; j += 4)
          *reinterpret_cast<float4 *>(dst + row * ld + c0 + j) =
              make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
    }
  }
}

template <typename T, int R, int D>
__global__ void __launch_bounds__(kPThreads, 2) project_kernel(ProjectParams p) {
  using PL = Plan<T, R, D>;
  constexpr bool TC = PL::TC;
  constexpr int RB = PL::RB, SR = PL::SR, LDB = PL::LDB, LDG = PL::LDG, SLOT = PL::SLOT;
  constexpr int EPV = Piece<T>::N;                     // elements per 16-byte piece
  constexpr int CPR = R * (int)sizeof(T) / 16;         // pieces per rank-r row
  constexpr int PPS = SR * CPR;                        // pieces per stage
  constexpr int PPT = (PPS + kPThreads - 1) / kPThreads;  // pieces per thread and stage
  constexpr int LPK = RB / 32;                         // lanes per key row: two 16-byte pieces each
  constexpr int RPP = kPThreads / LPK;                 // key rows per pass of the CTA
  constexpr int TE = R / 4, TG = TE * TE, NG = kPThreads / TG;  // Gram tiles, thread groups (fp32 path)
  constexpr int NGW = kPThreads / R;                   // thread groups of the weighted column sum
  constexpr uint32_t kTmemCols = 128;                  // two accumulators of 64 columns
  static_assert(SR % RPP == 0, "a stage is a whole number of passes");
  static_assert(!TC || SR <= 64, "a stage of rank-r rows must fit one operand tile");

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
  const int n_act = p.k + p.m;
  const int share = (n_act + n_streamers - 1) / n_streamers;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  // operand tiles first, on a 1024-byte boundary (the swizzle pattern is tied to the address bits)
  unsigned char *tiles = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
  float *sm = reinterpret_cast<float *>(tiles + PL::tile_bytes);
  float *qs = sm + PL::o_qs, *ks = sm + PL::o_ks;
  uint64_t *bars = reinterpret_cast<uint64_t *>(sm + PL::o_bars);  // [kRing] ring stages, then:
  uint64_t *mma_bar = bars + kRing;                                 // [2] the MMAs that read tile 0 / 1 have retired
  uint64_t *acc_bar = bars + kRing + 2;                             // every MMA issued so far has completed
  uint64_t *b_bar = bars + kRing + 3;                               // the MMAs of a right factor's Gram have completed
  float *slots = sm + PL::o_slots;                                  // solver CTA only: [n_streamers][SLOT]
  float *region = sm + PL::common_floats(csize == 1 ? 1 : (solver ? n_streamers : 0));
  // streaming buffers
  unsigned char *ring = reinterpret_cast<unsigned char *>(region + PL::s_ring);
  float *At = region + PL::s_At;
  float *S = region + PL::s_S;
  int32_t *pos_s = reinterpret_cast<int32_t *>(region + PL::s_pos);
  // solver buffers: behind the streaming buffers when this CTA does both jobs, else in their place
  float *sol = csize == 1 ? region + PL::stream_floats(share) : region;
  float *BQ = sol + PL::v_BQ, *BK = sol + PL::v_BK;
  float *GQ = sol + PL::v_GQ, *GQi = sol + PL::v_GQi, *GK = sol + PL::v_GK, *GKi = sol + PL::v_GKi;
  float *vec = sol + PL::v_vec, *misc = sol + PL::v_misc;
  float *qrhs = vec, *kbk = vec + R, *khat = vec + 2 * R, *qhat = vec + 3 * R, *knew = vec + 4 * R;
  float *rhs = vec + 5 * R, *tmpv = vec + 6 * R;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + PL::o_bars + 2 * (kRing + 4));
  const uint32_t tile0 = smem_addr(tiles), tile_zero = tile0 + 2 * kTileBytes;

  pdl_launch_dependents();
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kRing + 4; ++s) mbarrier_init(&bars[s], 1);
    mbarrier_init_fence();
  }
  uint32_t tmem_base = 0;
  if constexpr (TC) {
    for (int i = tid; i < 3 * kTileBytes / 16; i += kPThreads) reinterpret_cast<uint4 *>(tiles)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the zero fill is read by the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if constexpr (TC) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    tmem_base = *tmem_slot;
  }
  pdl_wait();

  // ---- streaming CTAs: request the first stages of their share at once --------------------------------
  const int srank = csize == 1 ? 0 : rank - 1;
  const int j_begin = min(n_act, srank * share);
  const int j_end = min(n_act, j_begin + share);
  const int nrows = streamer ? j_end - j_begin : 0;
  const int nstages = (nrows + SR - 1) / SR;
  const char *Kg = reinterpret_cast<const char *>(p.K_res) + ((int64_t)n * n_act + j_begin) * RB;
  if (streamer && tid == 0) {
    for (int s = 0; s < kRing && s < nstages; ++s) {
      const int rows_s = min(SR, nrows - s * SR);
      bulk_load(ring + s * kStageBytesK, Kg + (int64_t)s * SR * RB, (uint32_t)rows_s * RB, &bars[s]);
    }
  }
  {
    const T *qg = reinterpret_cast<const T *>(p.q) + (int64_t)n * D;
    const T *kg = reinterpret_cast<const T *>(p.k_new) + ((int64_t)b_idx * kv_heads + kvh) * D;
    for (int e = tid; e < D; e += kPThreads) {
      qs[e] = Elt<T>::to_float(qg[e]);
      ks[e] = Elt<T>::to_float(kg[e]);
    }
  }
  if (streamer) {
    const int32_t *tab = p.table + (int64_t)n * p.k;
    for (int i = tid; i < nrows; i += kPThreads) {
      const int j = j_begin + i;
      pos_s[i] = j == p.fuse_row ? p.position : (j < p.k ? tab[j] : p.lite_pos[j - p.k]);
    }
  }
  __syncthreads();

  bool timed_out = false;
  // ---- solver CTA: everything that does not depend on the active rows -----------------------------------
  if (solver && p.fuse_row >= 0) {  // fused ring write: 16-byte copies of the step's key and value
    constexpr int CH = D * (int)sizeof(T) / 16;
    const int64_t dst = ((int64_t)n * n_act + p.fuse_row) * D * (int64_t)sizeof(T);
    const int64_t src = ((int64_t)b_idx * kv_heads + kvh) * D * (int64_t)sizeof(T);
    if (tid < CH) st16(reinterpret_cast<char *>(p.K_res_w) + dst + tid * 16, ld16(reinterpret_cast<const char *>(p.k_new) + src + tid * 16));
    else if (tid < 2 * CH) st16(reinterpret_cast<char *>(p.V_res_w) + dst + (tid - CH) * 16,
                                ld16(reinterpret_cast<const char *>(p.v_new) + src + (tid - CH) * 16));
    if (n == 0 && tid == 2 * CH) p.lite_pos_w[p.fuse_row - p.k] = p.position;
  }
  if (solver) {
    const T *BQg = reinterpret_cast<const T *>(p.B_Q) + (int64_t)n * R * D;
    const T *BKg = reinterpret_cast<const T *>(p.B_K) + (int64_t)n * R * D;
    constexpr int PIECES = R * D / EPV;
    if constexpr (TC) {
      // B B^T on the tensor cores.  The contraction runs over the d columns of B, so the operand tile holds
      // B TRANSPOSED: tile row = column e of B, tile column = row a of B (one 64-row tile per 64 columns).
      // A thread turns each of its 16-byte pieces (8 neighbouring columns of one row) into 8 two-byte
      // stores.  Pieces are dealt out row-fastest (lane <-> row a, the lanes of a warp share the columns),
      // so that a warp's stores land in one 128-byte tile row: no bank conflicts.
      constexpr int PPTB = (PIECES + kPThreads - 1) / kPThreads;  // pieces per thread
      uint4 raw[2][PPTB];
#pragma unroll
      for (int w = 0; w < PPTB; ++w) {
        const int i = tid + w * kPThreads;
        const int a = i % R, e0 = (i / R) * EPV;
        raw[0][w] = i < PIECES ? ld16(BQg + (int64_t)a * D + e0) : make_uint4(0u, 0u, 0u, 0u);
        raw[1][w] = i < PIECES ? ld16(BKg + (int64_t)a * D + e0) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int which = 0; which < 2; ++which) {
#pragma unroll
        for (int w = 0; w < PPTB; ++w) {
          const int i = tid + w * kPThreads;
          const int a = i % R, e0 = (i / R) * EPV;
          if (i < PIECES) {
            const uint32_t words[4] = {raw[which][w].x, raw[which][w].y, raw[which][w].z, raw[which][w].w};
#pragma unroll
            for (int xx = 0; xx < EPV; ++xx) {
              const int e = e0 + xx, row = e & 63;
              const uint16_t bits = (uint16_t)(words[xx >> 1] >> ((xx & 1) * 16));
              *reinterpret_cast<uint16_t *>(tiles + (e >> 6) * kTileBytes + tile_chunk(row, a >> 3) + (a & 7) * 2) = bits;
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int t = 0; t < D / 64; ++t) gram_tile_mma(tile0 + t * kTileBytes, tile_zero, tmem_base + which * 64, t > 0);
          tc::umma_commit(b_bar);
        }
        // x B^T while the tensor core works: a warp per row of B, the lanes over its columns (the rows are
        // in L2 from the loads above)
        {
          const T *Bg = which == 0 ? BQg : BKg;
          const float *x = which == 0 ? qs : ks;
          float *xb = which == 0 ? qrhs : kbk;
          for (int a = warp; a < R; a += kPWarps) {
            float acc = 0.0f;
            for (int e = 2 * lane; e < D; e += 64) {
              const uint32_t w2 = *reinterpret_cast<const uint32_t *>(Bg + (int64_t)a * D + e);
              acc = fmaf(__uint_as_float(w2 << 16), x[e], acc);
              acc = fmaf(__uint_as_float(w2 & 0xFFFF0000u), x[e + 1], acc);
            }
            acc = warp_sum(acc);
            if (lane == 0) xb[a] = acc;
          }
        }
        if (!mbar_wait_bounded(b_bar, (uint32_t)which)) timed_out = true;  // the tiles are free again (and the sums complete)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      gram_from_tmem<R>(tmem_base, 0, GQ, LDG);
      gram_from_tmem<R>(tmem_base, 64, GK, LDG);
      // (nothing to clear in the tiles: B only wrote columns 0..r-1, and every stage of rank-r rows overwrites
      // columns 0..r-1 of all 64 rows)
      if (warp == kPWarps - 1) {
        float acc = 0.0f;
        for (int e = lane; e < D; e += 32) acc = fmaf(qs[e], ks[e], acc);
        acc = warp_sum(acc);
        if (lane == 0) misc[0] = acc;  // q k^T
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    } else {
#pragma unroll 2
      for (int i = tid; i < PIECES; i += kPThreads) {
        const int a = (i * EPV) / D, e = (i * EPV) % D;
        float fq[EPV], fk[EPV];
        Piece<T>::unpack(ld16(BQg + (int64_t)i * EPV), fq);
        Piece<T>::unpack(ld16(BKg + (int64_t)i * EPV), fk);
#pragma unroll
        for (int x = 0; x < EPV; x += 4) {
          *reinterpret_cast<float4 *>(BQ + a * LDB + e + x) = make_float4(fq[x], fq[x + 1], fq[x + 2], fq[x + 3]);
          *reinterpret_cast<float4 *>(BK + a * LDB + e + x) = make_float4(fk[x], fk[x + 1], fk[x + 2], fk[x + 3]);
        }
      }
      __syncthreads();
      float *part_sol = sol + PL::v_part;
      gram_bbt<R, D>(BQ, LDB, part_sol, GQ, LDG);  // B_Q B_Q^T
      gram_bbt<R, D>(BK, LDB, part_sol, GK, LDG);  // B_K B_K^T
      // q B_Q^T, k B_K^T: a warp per row, lanes over the columns; q k^T by the way
      for (int a = warp; a < 2 * R; a += kPWarps) {
        const float *Brow = (a < R ? BQ + a * LDB : BK + (a - R) * LDB);
        const float *x = a < R ? qs : ks;
        float acc = 0.0f;
        for (int e = 4 * lane; e < D; e += 128) {
          const float4 bv = *reinterpret_cast<const float4 *>(Brow + e);
          const float4 xv = *reinterpret_cast<const float4 *>(x + e);
          acc = fmaf(bv.x, xv.x, acc); acc = fmaf(bv.y, xv.y, acc); acc = fmaf(bv.z, xv.z, acc); acc = fmaf(bv.w, xv.w, acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) (a < R ? qrhs : kbk)[a < R ? a : a - R] = acc;
      }
      if (warp == kPWarps - 1) {
        float acc = 0.0f;
        for (int e = lane; e < D; e += 32) acc = fmaf(qs[e], ks[e], acc);
        acc = warp_sum(acc);
        if (lane == 0) misc[0] = acc;  // q k^T
      }
      __syncthreads();
    }
    for (int i = tid; i < R * LDG; i += kPThreads) GKi[i] = GK[i];
    __syncthreads();
    cta_spd_inverse<R>(GKi, LDG);  // (B_K B_K^T)^-1
    if (warp == 0) {  // k_hat0 = k B_K^T (B_K B_K^T)^-1, with one refinement step against B_K B_K^T itself
      for (int i = lane; i < R; i += 32) tmpv[i] = col_dot4<R>(GKi, LDG, i, kbk);
      __syncwarp();
      for (int i = lane; i < R; i += 32) rhs[i] = kbk[i] - col_dot4<R>(GK, LDG, i, tmpv);
      __syncwarp();
      for (int i = lane; i < R; i += 32) khat[i] = tmpv[i] + col_dot4<R>(GKi, LDG, i, rhs);
    }
  }

  // ---- streaming CTAs: their share of the active rows ------------------------------------------------------
  if (streamer) {
    const T *AK = reinterpret_cast<const T *>(p.A_K) + (int64_t)n * p.a_capacity * R;
    const int fuse_local = p.fuse_row - j_begin;  // the step's own key is not in K_res yet when the ring write is fused
    // this lane's slices of q: the two 16-byte pieces it reads of every key row
    const int lk = tid % LPK, rk = tid / LPK;
    float qa[EPV], qb[EPV];
#pragma unroll
    for (int e = 0; e < EPV; ++e) { qa[e] = qs[lk * EPV + e]; qb[e] = qs[D / 2 + lk * EPV + e]; }
    // gather pipeline: pieces of the rank-r rows, kAhead stages ahead, in registers
    uint4 pre[kAhead][PPT];
    auto fetch = [&](int stage, uint4 (&dst)[PPT]) {
#pragma unroll
      for (int w = 0; w < PPT; ++w) {
        const int pi = tid + w * kPThreads;
        const int row = stage * SR + pi / CPR;
        dst[w] = (pi < PPS && row < nrows) ? ld16(AK + (int64_t)pos_s[row] * R + (pi % CPR) * EPV) : make_uint4(0u, 0u, 0u, 0u);
      }
    };
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (u < nstages) fetch(u, pre[u]);
    }
    const int grp = tid / TG, ty = (tid % TG) / TE, tx = tid % TE;
    const int cw = tid % R, gw = tid / R;
    float acc[4][4], wacc = 0.0f;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][c] = 0.0f;

    for (int s0 = 0; s0 < nstages; s0 += kAhead) {
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int s = s0 + u;
        if (s < nstages) {  // CTA-uniform
          const int slot = s % kRing, buf = s & 1;
          const int rows_s = min(SR, nrows - s * SR);
          float *At_s = At + buf * SR * R;
          float *S_s = S + buf * SR;
          unsigned char *tile_s = tiles + buf * kTileBytes;
          // rank-r rows of this stage out of the registers; then ask for stage s + kAhead
          if constexpr (TC) {
            // the MMAs of stage s - 2 read this tile: they must have retired
            if (s >= 2 && !mbar_wait_bounded(&mma_bar[buf], (uint32_t)((s >> 1) - 1) & 1u)) timed_out = true;
#pragma unroll
            for (int w = 0; w < PPT; ++w) {
              const int pi = tid + w * kPThreads;
              if (pi < PPS) *reinterpret_cast<uint4 *>(tile_s + tile_chunk(pi / CPR, pi % CPR)) = pre[u][w];
            }
          } else {
#pragma unroll
            for (int w = 0; w < PPT; ++w) {
              const int pi = tid + w * kPThreads;
              if (pi < PPS) {
                float f[EPV];
                Piece<T>::unpack(pre[u][w], f);
                float *dst = At_s + (pi / CPR) * R + (pi % CPR) * EPV;
#pragma unroll
                for (int x = 0; x < EPV; x += 4) *reinterpret_cast<float4 *>(dst + x) = make_float4(f[x], f[x + 1], f[x + 2], f[x + 3]);
              }
            }
          }
          if (s + kAhead < nstages) fetch(s + kAhead, pre[u]);
          // s_j = q . K_j from the ring
          if (!mbar_wait_bounded(&bars[slot], (uint32_t)(s / kRing) & 1u)) timed_out = true;
          const unsigned char *Ks = ring + slot * kStageBytesK;
#pragma unroll
          for (int pass = 0; pass < SR / RPP; ++pass) {
            const int row = pass * RPP + rk;
            const uint4 va = *reinterpret_cast<const uint4 *>(Ks + row * RB + lk * 16);
            const uint4 vb = *reinterpret_cast<const uint4 *>(Ks + row * RB + RB / 2 + lk * 16);
            float fa[EPV], fb[EPV];
            Piece<T>::unpack(va, fa);
            Piece<T>::unpack(vb, fb);
            if (s * SR + row == fuse_local) {
#pragma unroll
              for (int e = 0; e < EPV; ++e) { fa[e] = ks[lk * EPV + e]; fb[e] = ks[D / 2 + lk * EPV + e]; }
            }
            float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
            for (int e = 0; e < EPV; ++e) { d0 = fmaf(fa[e], qa[e], d0); d1 = fmaf(fb[e], qb[e], d1); }
            float d = d0 + d1;
#pragma unroll
            for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
            if (lk == 0) S_s[row] = (row < rows_s && !timed_out) ? d : 0.0f;
          }
          if constexpr (TC) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tile stores above -> tensor-core reads
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          }
          __syncthreads();  // this stage's rank-r rows and scores are in place; its ring slot is free
          if (tid == 0) {
            if (s + kRing < nstages) {
              const int sn = s + kRing;
              const int rows_n = min(SR, nrows - sn * SR);
              bulk_load(ring + slot * kStageBytesK, Kg + (int64_t)sn * SR * RB, (uint32_t)rows_n * RB, &bars[slot]);
            }
            if constexpr (TC) {  // G += (rows of the stage)^T (rows of the stage)
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
              gram_tile_mma(tile0 + buf * kTileBytes, tile_zero, tmem_base, s > 0);
              tc::umma_commit(&mma_bar[buf]);
            }
          }
          if constexpr (TC) {
            // w += s_j a_j straight from the operand tile
#pragma unroll 4
            for (int row = gw; row < rows_s; row += NGW) {
              const __nv_bfloat16 a = *reinterpret_cast<const __nv_bfloat16 *>(tile_s + tile_chunk(row, cw >> 3) + (cw & 7) * 2);
              wacc = fmaf(S_s[row], __bfloat162float(a), wacc);
            }
          } else {
            // G += a_j^T a_j (4 x 4 tile per thread, the groups take every NG-th row), w += s_j a_j
#pragma unroll 4
            for (int row = grp; row < rows_s; row += NG) {
              const float4 r4 = *reinterpret_cast<const float4 *>(At_s + row * R + 4 * ty);
              const float4 c4 = *reinterpret_cast<const float4 *>(At_s + row * R + 4 * tx);
              const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
              for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[a][c] = fmaf(rr[a], cc[c], acc[a][c]);
            }
#pragma unroll 4
            for (int row = gw; row < rows_s; row += NGW) wacc = fmaf(S_s[row], At_s[row * R + cw], wacc);
          }
        }
      }
    }
    // fold the thread groups in group order (the key ring is free by now) and hand the sums to the solver
    __syncthreads();
    float *part = reinterpret_cast<float *>(ring);  // fp32 path: NG * R * R floats; then NGW * R
    float *partw = part + (TC ? 0 : NG * R * R);
    float *slot_dst = (csize == 1 ? slots : cluster.map_shared_rank(slots, 0)) + srank * SLOT;
    if constexpr (TC) {
      if (tid == 0) tc::umma_commit(acc_bar);
      partw[gw * R + cw] = wacc;
      if (nstages > 0 && !mbar_wait_bounded(acc_bar, 0u)) timed_out = true;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      timed_out = __syncthreads_or(timed_out ? 1 : 0) != 0;  // one decision for the CTA: the loads below are warp-wide
      if (nstages > 0 && !timed_out) {
        gram_from_tmem<R>(tmem_base, 0, slot_dst, R);
      } else {
        for (int i = tid; i < R * R; i += kPThreads) slot_dst[i] = 0.0f;
      }
    } else {
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) part[grp * R * R + (4 * ty + a) * R + 4 * tx + c] = acc[a][c];
      partw[gw * R + cw] = wacc;
      __syncthreads();
      for (int i = tid; i < R * R / 4; i += kPThreads) {
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          const float4 v = reinterpret_cast<const float4 *>(part + g * R * R)[i];
          s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
        }
        reinterpret_cast<float4 *>(slot_dst)[i] = s4;
      }
    }
    if (tid < R) {
      float s1 = 0.0f;
#pragma unroll
      for (int g = 0; g < NGW; ++g) s1 += partw[g * R + tid];
      slot_dst[R * R + tid] = timed_out ? 0.0f : s1;
    }
  }
  if (timed_out && tid == 0) atomicExch(p.status, (int32_t)LRQK_ETIMEOUT);

  if constexpr (TC) asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();  // every streaming CTA's sums are in the solver's shared memory
  if constexpr (TC) {
    if (warp == 0) {  // nothing of this CTA touches tensor memory any more
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
  }
  if (!solver) return;

  // ---- solver: B_Q B_Q^T + A^T A, q B_Q^T + (q K^T) A, then the alternating solves -------------------------------
  for (int i = tid; i < R * R; i += kPThreads) {
    float s = 0.0f;
    for (int c = 0; c < n_streamers; ++c) s += slots[c * SLOT + i];
    const int idx = (i / R) * LDG + i % R;
    const float g = fmaf(p.lam_act, s, GQ[idx]);
    GQ[idx] = g;
    GQi[idx] = g;
  }
  if (tid < R) {
    float s = 0.0f;
    for (int c = 0; c < n_streamers; ++c) s += slots[c * SLOT + R * R + tid];
    qrhs[tid] = fmaf(p.lam_act, s, qrhs[tid]);
  }
  __syncthreads();
  cta_spd_inverse<R>(GQi, LDG);

  float *ws = p.ws + (int64_t)n * p.max_iter * (2 * R + 2);
  if (warp == 0) {
    const float qk = p.lam_own * misc[0];
    for (int it = 0; it < p.max_iter; ++it) {
      // q_hat = (qrhs + qk * k_hat)(GQ + lam_own k_hat^T k_hat)^-1
      for (int i = lane; i < R; i += 32) rhs[i] = fmaf(qk, khat[i], qrhs[i]);
      __syncwarp();
      warp_rank1_solve<R>(GQ, GQi, LDG, khat, p.lam_own, rhs, qhat, tmpv);
      // k_hat' = (kbk + qk * q_hat)(GK + lam_own q_hat^T q_hat)^-1
      for (int i = lane; i < R; i += 32) rhs[i] = fmaf(qk, qhat[i], kbk[i]);
      __syncwarp();
      warp_rank1_solve<R>(GK, GKi, LDG, qhat, p.lam_own, rhs, knew, tmpv);
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
    if (n == 0 && lane == 0 && p.clear_word) *p.clear_word = 0;
  }
}

struct UpdateParams {
  UpdateArgs u;
  int32_t *clear_word;  // optional: set to zero by the kernel
};

template <typename T, int R, int D>
__global__ void __launch_bounds__(D) update_kernel(UpdateParams p) {
  __shared__ float delta[8];
  extern __shared__ __align__(16) float sh[];  // update_head_smem_floats(R, D)
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int chosen = update_chosen<R>(p.u, delta);
  if (n == 0 && threadIdx.x == 0) {
    if (p.u.iters_out) *p.u.iters_out = chosen + 1;
    if (p.clear_word) *p.clear_word = 0;
  }
  update_head<T, R>(p.u, n, chosen, sh);
}

template <typename T, int R, int D>
size_t project_smem_bytes(int csize, int share_rows) {
  using PL = Plan<T, R, D>;
  const int n_streamers = csize == 1 ? 1 : csize - 1;
  const size_t stream = (size_t)PL::stream_floats(share_rows);
  const size_t solve = (size_t)PL::solver_floats;
  size_t floats;
  if (csize == 1) floats = PL::common_floats(1) + stream + solve;
  else {
    const size_t a = (size_t)PL::common_floats(n_streamers) + solve, b = (size_t)PL::common_floats(0) + stream;
    floats = a > b ? a : b;
  }
  return sizeof(float) * floats + PL::tile_bytes + 1024 + 128;  // slack for the 1024-byte alignment of the tiles
}

// A lower bound of how many clusters of `csize` CTAs of the projection kernel the current device keeps resident at
// once (a cluster must fit inside one GPC, so this is not simply CTA slots / csize).  Asked of the runtime once per
// (kernel, cluster size, shared-memory size, device); 0 when it cannot be told.
template <typename T, int R, int D>
SmemOptIn &project_opt_in() {
  static SmemOptIn o;  // one record of the kernel's shared-memory attribute per device, shared by launch and query
  return o;
}

template <typename T, int R, int D>
int project_resident_clusters(int csize, size_t smem) {
  struct Entry { size_t smem; int n; };  // the answer for the last shared-memory size asked about
  static std::mutex mu;
  static Entry cache[kMaxDevices][9] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || csize < 1 || csize > 8) { cudaGetLastError(); return 0; }
  std::lock_guard<std::mutex> lock(mu);
  Entry &c = cache[dev][csize];
  if (c.n == 0 || c.smem != smem) {
    auto kern = project_kernel<T, R, D>;
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize, 1, 1);
    cfg.blockDim = dim3(kPThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)csize; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = project_opt_in<T, R, D>().ensure(kern, smem);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    // The runtime's figure is for one CTA of the cluster per SM (15 clusters of 8 on a 148-SM part).  Where an SM
    // holds two CTAs of this kernel it says nothing useful (32 clusters of 8 are resident at once there): -2.
    // (two CTAs: by shared memory -- the kernel's register bound is set for two)
    if (e == cudaSuccess && 2 * (smem + 1024) <= 227 * 1024) n = -2;
    if (e != cudaSuccess) { cudaGetLastError(); n = -1; }
    c.smem = smem;
    c.n = n > 0 ? n : (n == -2 ? -2 : -1);
  }
  return c.n > 0 ? c.n : 0;  // 0: not known
}

// Clusters: one solver CTA plus streaming CTAs.  The cluster grows (2, 4, 8 CTAs) while every streaming
// CTA keeps at least two ring stages of rows and the grid stays within the CTAs that are resident at
// once (two per SM); rank 64 keeps to clusters of 2..4 (its solver holds 16 KiB of partial sums per
// streaming CTA, and solver and streaming buffers together exceed one CTA's shared memory).  Where only one
// CTA fits an SM (rank 64) the runtime knows how many clusters are resident at once, and the cluster shrinks
// until every head's is: a cluster that has to wait for a place starts when the first streaming CTAs leave
// and ends long after all the others (40 heads: clusters of 3, all resident, instead of 33 of 40 clusters of 4).
template <typename T, int R, int D>
size_t project_smem_for(int csize, int n_act) {
  const int n_streamers = csize == 1 ? 1 : csize - 1;
  return project_smem_bytes<T, R, D>(csize, (n_act + n_streamers - 1) / n_streamers);
}

template <typename T, int R, int D>
int plan_cluster(int n_heads, int n_act) {
  constexpr int SR = Plan<T, R, D>::SR;
  const int max_c = R >= 64 ? 4 : 8;
  const int min_c = R >= 64 ? 2 : 1;
  int csize = min_c;
  while (csize < max_c && n_heads * csize * 2 <= 2 * kNumSMs && n_act / (csize * 2 - 1) >= 2 * SR) csize *= 2;
  while (csize > min_c) {
    const int resident = project_resident_clusters<T, R, D>(csize, project_smem_for<T, R, D>(csize, n_act));
    if (resident <= 0 || n_heads <= resident) break;
    --csize;
  }
  return csize;
}

template <typename T, int R, int D>
int launch(const lrqk_layer *L, ProjectParams pp, const UpdateParams &up, cudaStream_t stream, bool with_update,
           bool with_project) {
  const int n_heads = L->bsz * L->q_heads;
  const int n_act = L->k + L->m;
  const int csize = plan_cluster<T, R, D>(n_heads, n_act);
  const int n_streamers = csize == 1 ? 1 : csize - 1;
  const int share = (n_act + n_streamers - 1) / n_streamers;
  const size_t smem = project_smem_bytes<T, R, D>(csize, share);
  if (smem > 227 * 1024) return LRQK_EUNSUPPORTED;
  if (with_project) {
    auto kern = project_kernel<T, R, D>;
    LRQK_CUDA_TRY((project_opt_in<T, R, D>().ensure(kern, smem)));
    LRQK_CUDA_TRY(launch_dependent(kern, dim3(csize, n_heads, 1), dim3(kPThreads), smem, stream, csize, pp));
  }
  if (with_update) {
    constexpr size_t usmem = sizeof(float) * (size_t)update_head_smem_floats(R, D);
    static SmemOptIn opt_in_u;
    if (usmem > 48 * 1024) LRQK_CUDA_TRY(opt_in_u.ensure(update_kernel<T, R, D>, usmem));
    LRQK_CUDA_TRY(launch_dependent(update_kernel<T, R, D>, dim3(n_heads), dim3(D), usmem, stream, 0, up));
  }
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

template <typename T, int D>
int dispatch_r(const lrqk_layer *L, const ProjectParams &pp, const UpdateParams &up, cudaStream_t stream, bool with_update,
               bool with_project) {
  switch (L->r) {
    case 8: return launch<T, 8, D>(L, pp, up, stream, with_update, with_project);
    case 16: return launch<T, 16, D>(L, pp, up, stream, with_update, with_project);
    case 32: return launch<T, 32, D>(L, pp, up, stream, with_update, with_project);
    case 64: return launch<T, 64, D>(L, pp, up, stream, with_update, with_project);
    default: return LRQK_EUNSUPPORTED;
  }
}

}  // namespace
}  // namespace lrqk

// Workspace: the iterates of every head, [N][max_iter][2r + 2] floats, then one int32 status word
// (LRQK_ETIMEOUT if a bounded wait of the kernel ran out; 0 otherwise) on a 16-byte boundary.
static size_t project_iterates_bytes(const lrqk_layer *L, int32_t it) {
  return (sizeof(float) * (size_t)L->bsz * L->q_heads * it * (2 * L->r + 2) + 15) / 16 * 16;
}

extern "C" size_t lrqk_decode_project_update_workspace_bytes(const lrqk_layer *L, int32_t max_iter) {
  if (!L || max_iter < 0) return 0;
  return project_iterates_bytes(L, max_iter < 1 ? 1 : max_iter) + 16;
}

extern "C" int32_t *lrqk_decode_project_update_status_word(const lrqk_layer *L, int32_t max_iter, void *workspace) {
  if (!L || !workspace || max_iter < 0) return nullptr;
  return reinterpret_cast<int32_t *>(reinterpret_cast<char *>(workspace) + project_iterates_bytes(L, max_iter < 1 ? 1 : max_iter));
}

// The two halves as separate calls.  (The fused step runs the first as its own kernel and applies the second
// inside the scoring kernel.)
extern "C" int lrqk_decode_project(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter,
                                   int64_t append_row, void *q_hat, void *workspace, lrqk_stream_t stream) {
  lrqk::UpdateArgs unused;
  return lrqk::project_update_enqueue(L, q, k_new, max_iter, 0.0f, append_row, q_hat, nullptr, workspace, nullptr,
                                      lrqk::as_stream(stream), nullptr, -1, &unused);
}

extern "C" int lrqk_decode_update(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter, float tol,
                                  int64_t append_row, void *q_hat, int32_t *iters_out, void *workspace,
                                  lrqk_stream_t stream) {
  return lrqk::project_update_enqueue(L, q, k_new, max_iter, tol, append_row, q_hat, iters_out, workspace, nullptr,
                                      lrqk::as_stream(stream), nullptr, -1, nullptr, true);
}

extern "C" int lrqk_decode_project_update(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter,
                                          float tol, int64_t append_row, void *q_hat, int32_t *iters_out,
                                          void *workspace, lrqk_stream_t stream) {
  return lrqk::project_update_enqueue(L, q, k_new, max_iter, tol, append_row, q_hat, iters_out, workspace, nullptr,
                                      lrqk::as_stream(stream), nullptr, -1, nullptr);
}

int lrqk::project_update_enqueue(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter, float tol,
                                 int64_t append_row, void *q_hat, int32_t *iters_out, void *workspace,
                                 int32_t *clear_word, cudaStream_t s, const void *v_new, int32_t lite_slot,
                                 UpdateArgs *deferred, bool update_only) {
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
  pp.lam_own = L->weights[2]; pp.lam_act = L->weights[3];  // lambda_dec_q, lambda_dec_k (:1535-1536 -> :433-446)
  pp.ws = reinterpret_cast<float *>(workspace);
  pp.status = reinterpret_cast<int32_t *>(reinterpret_cast<char *>(workspace) + project_iterates_bytes(L, max_iter));
  pp.v_new = v_new; pp.K_res_w = L->K_res; pp.V_res_w = L->V_res; pp.lite_pos_w = L->lite_pos;
  pp.fuse_row = -1; pp.position = (int32_t)append_row;
  if (v_new) {
    if (lite_slot < 0 || lite_slot >= L->m || !L->V_res) return LRQK_EINVAL;
    pp.fuse_row = L->k + lite_slot;
  }
  UpdateParams up;
  up.u.A_K = L->A_K; up.u.B_Q = L->B_Q; up.u.B_K = L->B_K; up.u.q = q; up.u.k_new = k_new;
  up.u.ws = pp.ws; up.u.q_hat = q_hat; up.u.iters_out = iters_out;
  up.u.a_capacity = L->a_capacity; up.u.append_row = append_row;
  up.u.q_heads = L->q_heads; up.u.groups = pp.groups; up.u.max_iter = max_iter; up.u.n_heads = pp.n_heads;
  up.u.head_dim = L->head_dim;
  up.u.tol = tol;
  up.clear_word = clear_word;
  pp.clear_word = nullptr;
  const bool with_update = deferred == nullptr;
  if (deferred) {  // the caller's next kernel applies the update itself; this kernel clears the word instead
    *deferred = up.u;
    pp.clear_word = clear_word;
  }
  if (L->head_dim == 128) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, return (dispatch_r<T, 128>(L, pp, up, s, with_update, !update_only)));
  } else if (L->head_dim == 64) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, return (dispatch_r<T, 64>(L, pp, up, s, with_update, !update_only)));
  }
  return LRQK_EUNSUPPORTED;
}
