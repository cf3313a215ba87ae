// Proxy scoring over the rank-r key factors fused with a cluster-wide radix top-k.
//
// One thread-block cluster per (batch, query head).  The candidate rows of A_K are cut into
// one contiguous segment per CTA.  Each CTA streams its segment once from HBM with 32-byte
// evict-first loads, forms the fp32 dot product with q_hat and keeps the scores -- as
// order-preserving 32-bit keys -- in shared memory; they never travel to global memory.  The
// k-th largest key is then found by a three-pass (11+11+10 bit) radix select whose per-CTA
// histograms are summed through distributed shared memory, and the selected positions are
// written in ascending order by an ordered compaction (block scans inside a CTA, a DSMEM
// exchange of counts between CTAs).  Of equal scores the lower position wins.
//
// Summation order of a score (fixed, so results are reproducible): the r columns are split
// over `lanes = row_bytes / vector_bytes` lanes, each lane sums its run left to right with
// fused multiply-adds starting from zero, and the lanes are combined by a butterfly
// (partner distance 1, 2, 4, ...).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace lrqk {
namespace {

constexpr int kThreads = 512;
constexpr int kTile = 4 * kThreads;  // keys handled per compaction tile
constexpr int kBins0 = 2048;         // 11-bit digits for passes 0 and 1, 10 bits for pass 2
constexpr int kUnroll = 4;
constexpr int kCandPerWarp = 128;      // per-warp list of keys still matching the radix prefix
constexpr int kCandCap = kCandPerWarp * (kThreads / 32);

template <int VB> struct Vec;
template <> struct Vec<32> {
  uint32_t w[8];
  __device__ __forceinline__ void load(const void *p) {
    asm volatile("ld.global.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p));
  }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = 0;
  }
};
template <> struct Vec<16> {
  uint32_t w[4];
  __device__ __forceinline__ void load(const void *p) {
    uint4 v = ld_stream16(p);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  }
  __device__ __forceinline__ void zero() { w[0] = w[1] = w[2] = w[3] = 0; }
};

// Unpack the words of a vector into floats.
template <typename T, int NW> struct Unpack;
template <int NW> struct Unpack<float, NW> {
  static constexpr int kElts = NW;
  __device__ static __forceinline__ void run(const uint32_t (&w)[NW], float (&f)[NW]) {
#pragma unroll
    for (int i = 0; i < NW; ++i) f[i] = __uint_as_float(w[i]);
  }
};
template <int NW> struct Unpack<__nv_bfloat16, NW> {
  static constexpr int kElts = 2 * NW;
  __device__ static __forceinline__ void run(const uint32_t (&w)[NW], float (&f)[2 * NW]) {
#pragma unroll
    for (int i = 0; i < NW; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
};

struct ScoreTopkParams {
  const void *A_K;      // [N, a_capacity, R]
  const void *q_hat;    // [N, R]
  int64_t a_capacity;
  int64_t candidates;
  int32_t k;
  int32_t seg_len;      // rows per CTA, multiple of kTile
  int32_t *wanted;      // [N, k]
  float *scores_out;    // optional [N, scores_stride]
  int64_t scores_stride;
};

// Exclusive block scan of one 32-bit value per thread (kThreads threads); returns the
// exclusive prefix and, through `total`, the block sum.  `scratch` holds 17 words.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t *scratch, uint32_t &total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = lane < (kThreads / 32) ? scratch[lane] : 0;
    uint32_t winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t t = __shfl_up_sync(0xFFFFFFFFu, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < (kThreads / 32)) scratch[lane] = winc - w;  // exclusive warp offsets
    if (lane == 31) scratch[16] = winc;                     // block total
  }
  __syncthreads();
  const uint32_t res = scratch[warp] + inc - v;
  total = scratch[16];
  __syncthreads();  // scratch may be reused right away
  return res;
}

// Keys live in shared memory with one pad word per 32 so that both access patterns used below
// (thread-strided and one contiguous run per thread) are free of bank conflicts.
__device__ __forceinline__ int phys(int i) { return i + (i >> 5); }

// Find the bin that holds the `need`-th largest key given cluster-wide bin totals in `tot_hist`
// (kBins0 words, larger bin = larger keys).  Returns through bcast[0] the bin, bcast[1] the
// count still needed inside that bin.  All threads must call.
__device__ __forceinline__ void pick_bin(const uint32_t *tot_hist, uint32_t need, uint32_t *scratch,
                                         uint32_t *bcast) {
  const int tid = threadIdx.x;
  const uint4 x = *reinterpret_cast<const uint4 *>(tot_hist + 4 * tid);
  const uint32_t tot[4] = {x.x, x.y, x.z, x.w};
  const uint32_t mine = tot[0] + tot[1] + tot[2] + tot[3];
  uint32_t all;
  const uint32_t below_incl = block_exclusive_scan(mine, scratch, all) + mine;
  uint32_t above = all - below_incl;  // keys in bins above this thread's four bins
  if (above < need && need <= above + mine) {
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      if (above + tot[j] >= need) {
        bcast[0] = (uint32_t)(4 * tid + j);
        bcast[1] = need - above;
        break;
      }
      above += tot[j];
    }
  }
  __syncthreads();
}

template <typename T, int R>
__global__ void __launch_bounds__(kThreads, 2) score_topk_kernel(ScoreTopkParams p) {
  constexpr int RB = R * (int)sizeof(T);          // bytes per row
  constexpr int VB = RB >= 32 ? 32 : 16;          // bytes per lane
  constexpr int LPR = RB / VB;                    // lanes per row
  constexpr int NW = VB / 4;                      // 32-bit words per lane
  constexpr int EPL = Unpack<T, NW>::kElts;       // elements per lane
  constexpr int RPI = kThreads / LPR;             // rows per CTA-wide load
  static_assert(kTile % (RPI * kUnroll) == 0, "tile must be a whole number of unrolled loads");

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int csize = (int)cluster.num_blocks();
  const int n = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  extern __shared__ __align__(16) uint32_t smem[];
  uint32_t *keys = smem;                                    // [seg_len + seg_len/32], padded
  uint32_t *hloc = keys + p.seg_len + (p.seg_len >> 5);     // [kBins0] this CTA's histogram of the pass
  uint32_t *htot = hloc + kBins0;                           // [2][kBins0] cluster totals (peers add into them)
  uint32_t *cand = htot + 2 * kBins0;                       // [kCandCap] local indices still matching the prefix
  uint32_t *scratch = cand + kCandCap;                      // [32]
  uint32_t *bcast = scratch + 32;                           // [8]  {bin, need, n_cand}
  uint32_t *cnts = bcast + 8;                               // [16][2] (greater, equal) per rank, written by peers
  uint32_t *wcount = cnts + 32;                             // [16] candidates seen by each warp

  for (int i = tid; i < 3 * kBins0; i += kThreads) hloc[i] = 0;
  if (tid < 8) bcast[tid] = 0;
  __syncthreads();
  cluster.barrier_arrive();  // peers may add into my totals once they have seen this

  // ---- streaming pass: scores -> keys in shared memory, pass-0 histogram on the fly -------
  const int64_t seg_begin = (int64_t)rank * p.seg_len;
  const int lane_in_row = tid % LPR;
  const int row_in_iter = tid / LPR;
  float qf[EPL];
  {
    const T *qh = reinterpret_cast<const T *>(p.q_hat) + (int64_t)n * R + lane_in_row * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) qf[e] = Elt<T>::to_float(qh[e]);
  }
  const char *base = reinterpret_cast<const char *>(p.A_K) + ((int64_t)n * p.a_capacity) * RB + lane_in_row * VB;
  int64_t seg_rows = p.candidates - seg_begin;   // rows of this segment that hold candidates
  if (seg_rows < 0) seg_rows = 0;
  if (seg_rows > p.seg_len) seg_rows = p.seg_len;
  const int n_iter_rows = (int)((seg_rows + RPI * kUnroll - 1) / (RPI * kUnroll)) * (RPI * kUnroll);

  for (int it = 0; it < n_iter_rows; it += RPI * kUnroll) {
    Vec<VB> v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int local = it + u * RPI + row_in_iter;
      if (local < seg_rows) v[u].load(base + (seg_begin + local) * RB);
      else v[u].zero();
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int local = it + u * RPI + row_in_iter;
      float a[EPL];
      Unpack<T, NW>::run(v[u].w, a);
      float acc = 0.0f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc = fmaf(a[e], qf[e], acc);
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
      if (lane_in_row == 0) {
        uint32_t key = 0;
        if (local < seg_rows) {
          key = order_key(acc);
          atomicAdd(&hloc[key >> 21], 1u);
          if (p.scores_out) p.scores_out[(int64_t)n * p.scores_stride + seg_begin + local] = acc;
        }
        keys[phys(local)] = key;
      }
    }
  }
  for (int i = n_iter_rows + tid; i < p.seg_len; i += kThreads) keys[phys(i)] = 0;  // padding sorts last
  __syncthreads();
  cluster.barrier_wait();

  // ---- radix select of the k-th largest key over the whole cluster ---------------------------
  // Three passes (11 + 11 + 10 bits).  Each CTA adds the non-zero bins of its histogram into
  // every peer's total through distributed shared memory, so that after one cluster barrier each
  // CTA finds the digit locally.  Passes 1 and 2 only visit the keys that matched so far.
  uint32_t prefix = 0;
  uint32_t need = (uint32_t)p.k;
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    const int bits = pass == 2 ? 10 : 11;
    const uint32_t dmask = (1u << bits) - 1;
    if (pass == 1) {
      // candidates: keys whose top 11 bits equal the chosen bin; every warp keeps a private list
      // (position counter in a register, slots handed out by ballot) so that no atomic is shared
      uint32_t mine_n = 0;
      uint32_t *wl = cand + warp * kCandPerWarp;
      for (int i = tid; i < p.seg_len; i += kThreads) {
        const uint32_t key = keys[phys(i)];
        const bool hit = (key >> 21) == prefix;
        const uint32_t bal = __ballot_sync(0xFFFFFFFFu, hit);
        if (hit) {
          atomicAdd(&hloc[(key >> shift) & dmask], 1u);
          const uint32_t at = mine_n + __popc(bal & ((1u << lane) - 1));
          if (at < (uint32_t)kCandPerWarp) wl[at] = (uint32_t)i;
        }
        mine_n += __popc(bal);
      }
      if (lane == 0) wcount[warp] = mine_n;
      __syncthreads();
    } else if (pass == 2) {
      const uint32_t mine_n = wcount[warp];
      bool overflow = false;
      for (int w = 0; w < kThreads / 32; ++w) overflow |= wcount[w] > (uint32_t)kCandPerWarp;
      if (!overflow) {
        const uint32_t *wl = cand + warp * kCandPerWarp;
        for (uint32_t c = lane; c < mine_n; c += 32) {
          const uint32_t key = keys[phys((int)wl[c])];
          if ((key >> 10) == prefix) atomicAdd(&hloc[key & dmask], 1u);
        }
      } else {  // some warp met more matches than its list holds: visit every key
        for (int i = tid; i < p.seg_len; i += kThreads) {
          const uint32_t key = keys[phys(i)];
          if ((key >> 10) == prefix) atomicAdd(&hloc[key & dmask], 1u);
        }
      }
      __syncthreads();
    }
    uint32_t *ht = htot + (pass & 1) * kBins0;
#pragma unroll
    for (int j = 0; j < kBins0 / kThreads; ++j) {
      const int b = tid + j * kThreads;
      const uint32_t v = hloc[b];
      if (v) {
        hloc[b] = 0;
        for (int c = 0; c < csize; ++c) atomicAdd(cluster.map_shared_rank(ht, c) + b, v);
      }
    }
    cluster.sync();  // every CTA's contribution has landed
    pick_bin(ht, need, scratch, bcast);
    prefix = (prefix << bits) | bcast[0];
    need = bcast[1];
    if (pass == 0) {  // totals[0] is used again by pass 2; peers add to it only after the next barrier
#pragma unroll
      for (int j = 0; j < kBins0 / kThreads; ++j) ht[tid + j * kThreads] = 0;
    }
    __syncthreads();
  }
  const uint32_t T_key = prefix;       // the k-th largest key
  const uint32_t need_ties = need;     // how many keys equal to it are taken (lowest positions)

  // ---- ordered compaction: one contiguous run of keys per thread ------------------------------
  const int per = p.seg_len / kThreads;
  uint32_t cg_ = 0, ce_ = 0;
#pragma unroll 4
  for (int j = 0; j < per; ++j) {
    const uint32_t key = keys[phys(tid * per + j)];
    cg_ += key > T_key;
    ce_ += key == T_key;
  }
  uint32_t cta_total;
  const uint32_t ex = block_exclusive_scan(cg_ | (ce_ << 16), scratch, cta_total);  // counts fit 16 bits
  if (tid < csize) {  // tell every rank how many keys this CTA holds above / at the threshold
    uint32_t *rc = cluster.map_shared_rank(cnts, tid);
    rc[2 * rank] = cta_total & 0xFFFFu;
    rc[2 * rank + 1] = cta_total >> 16;
  }
  cluster.sync();
  uint32_t out_base = 0, tie_base = 0, quota = 0;
  for (int c = 0; c <= rank; ++c) {
    const uint32_t g = cnts[2 * c], e = cnts[2 * c + 1];
    const uint32_t left = need_ties > tie_base ? need_ties - tie_base : 0;
    const uint32_t q = e < left ? e : left;
    if (c < rank) { out_base += g + q; tie_base += e; }
    else quota = q;
  }
  int32_t *out = p.wanted + (int64_t)n * p.k;
  uint32_t gb = ex & 0xFFFFu, eb = ex >> 16;
#pragma unroll 4
  for (int j = 0; j < per; ++j) {
    const int i = tid * per + j;
    const uint32_t key = keys[phys(i)];
    const bool is_g = key > T_key, is_e = key == T_key;
    if (is_g || (is_e && eb < quota)) {
      const uint32_t pos = out_base + gb + (eb < quota ? eb : quota);
      if (pos < (uint32_t)p.k) out[pos] = (int32_t)(seg_begin + i);
    }
    gb += is_g;
    eb += is_e;
  }
  // no peer touches this CTA's shared memory after the last cluster barrier above
}

template <typename T, int R>
int launch_score_topk(const ScoreTopkParams &p, int n_heads, int csize, cudaStream_t stream) {
  const size_t smem = ((size_t)p.seg_len + (p.seg_len >> 5) + 3 * kBins0 + kCandCap + 32 + 8 + 32 + 16) * sizeof(uint32_t);
  auto kern = score_topk_kernel<T, R>;
  static size_t smem_set = 0;
  static bool nonportable_set = false;
  if (smem > smem_set) {
    LRQK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    smem_set = smem;
  }
  if (csize > 8 && !nonportable_set) {
    LRQK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    nonportable_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(csize, n_heads, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  LRQK_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return LRQK_OK;
}

template <typename T>
int dispatch_rank(int r, const ScoreTopkParams &p, int n_heads, int csize, cudaStream_t stream) {
  switch (r) {
    case 8: return launch_score_topk<T, 8>(p, n_heads, csize, stream);
    case 16: return launch_score_topk<T, 16>(p, n_heads, csize, stream);
    case 32: return launch_score_topk<T, 32>(p, n_heads, csize, stream);
    case 64: return launch_score_topk<T, 64>(p, n_heads, csize, stream);
    default: return LRQK_EUNSUPPORTED;
  }
}

}  // namespace

// Cluster size and segment length for `candidates` rows per head and n_heads heads.
// The keys of a segment must fit in shared memory; beyond that, more CTAs per head are used
// while the grid stays within about two resident CTAs per SM.
int plan_score_topk(int64_t candidates, int n_heads, int *csize_out, int *seg_len_out) {
  const int64_t max_seg = 45056;  // 176 KiB of keys next to the histograms
  int best = -1;
  for (int cs = 1; cs <= 16; cs *= 2) {
    const int64_t seg = ceil_div64(ceil_div64(candidates, cs), kTile) * kTile;
    if (seg > max_seg) continue;
    if (best < 0) { best = cs; continue; }  // smallest cluster whose segment fits
    // grow the cluster (portable sizes only) while the whole grid stays resident at once
    // (two 80-KiB CTAs per SM) and every CTA still gets at least one full tile of rows
    if (cs <= 8 && (int64_t)n_heads * cs <= 2 * kNumSMs && ceil_div64(candidates, cs) >= kTile) best = cs;
  }
  if (best < 0) return LRQK_EUNSUPPORTED;
  *csize_out = best;
  *seg_len_out = (int)(ceil_div64(ceil_div64(candidates, best), kTile) * kTile);
  return LRQK_OK;
}

}  // namespace lrqk

extern "C" int lrqk_score_topk(const lrqk_layer *L, const void *q_hat, int64_t candidates, int32_t *wanted,
                               float *scores_out, int64_t scores_stride, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!q_hat || !wanted || !L->A_K) return LRQK_EINVAL;
  if (candidates > L->a_capacity) return LRQK_ECAPACITY;
  if (candidates <= L->k) return LRQK_EINVAL;
  if (scores_out && scores_stride < candidates) return LRQK_EINVAL;
  const int n_heads = L->bsz * L->q_heads;
  if (n_heads > 65535) return LRQK_EUNSUPPORTED;
  ScoreTopkParams p;
  p.A_K = L->A_K;
  p.q_hat = q_hat;
  p.a_capacity = L->a_capacity;
  p.candidates = candidates;
  p.k = L->k;
  p.wanted = wanted;
  p.scores_out = scores_out;
  p.scores_stride = scores_stride;
  int csize = 1, seg_len = 0;
  rc = plan_score_topk(candidates, n_heads, &csize, &seg_len);
  if (rc != LRQK_OK) return rc;
  p.seg_len = seg_len;
  LRQK_DISPATCH_DTYPE(L->dtype, T, return dispatch_rank<T>(L->r, p, n_heads, csize, as_stream(stream)));
  return LRQK_EUNSUPPORTED;
}
