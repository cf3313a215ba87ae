// Proxy scoring over the rank-r key factors fused with a cluster-wide radix top-k.
//
// One thread-block cluster per (batch, query head), one CTA of 1024 threads per SM.  The
// candidate rows of A_K are cut into one contiguous segment per CTA.  Each CTA streams its
// segment once from HBM with 32-byte evict-first loads, forms the fp32 dot product with q_hat
// and keeps the scores -- as order-preserving 32-bit keys -- in shared memory; they never
// travel to global memory.  The k-th largest key is then found by a three-pass (11+11+10 bit)
// radix select: every CTA builds the histogram of its own keys and exchanges it with its peers
// through distributed shared memory -- added into a cluster-wide histogram kept by every CTA where
// few bins are occupied, read from the peers where nearly all are -- so that after ONE cluster
// barrier per pass each CTA knows both the cluster totals (which digit holds the k-th key) and
// how many of the larger keys sit in lower-ranked CTAs (where its own output starts).  No further
// exchange is needed:
// every thread owns a contiguous run of keys, walks it once after the first pass (two bit masks:
// "above the digit", "equal to it"), and the later passes and the ordered, ascending compaction
// only revisit the marked keys.  Of equal scores the lower position wins.
//
// With few heads that plan leaves most SMs idle (a head spans at most 8 CTAs).  Then the work is cut
// differently: a first kernel streams A_K over ALL SMs -- work items of 2048 rows dealt out evenly,
// whatever head they belong to -- and writes the keys to a workspace that stays in L2 (4 bytes per
// candidate row); the select kernel then runs unchanged except that its CTAs fill their key segments from
// that workspace instead of from A_K.  Scores, keys and therefore the selection are bit-identical in
// both plans.
//
// Summation order of a score (fixed, so results are reproducible): the r columns are split
// over `lanes = max(1, row_bytes / 64)` lanes; each lane sums the even and the odd columns of its
// run separately, left to right with fused multiply-adds starting from zero (the two sums share
// one packed fp32x2 instruction), adds the two, and the lanes are combined by a butterfly
// (partner distance 1, 2, 4, ...).
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"
#include "slot_diff.cuh"
#include "update_head.cuh"

namespace cg = cooperative_groups;

namespace lrqk {
namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kBins = 2048;          // 11-bit digits for passes 0 and 1, 10 bits for pass 2
constexpr int kGranule = 4096;       // segment lengths are multiples of this many rows (4 per thread)
constexpr int kMaxSeg = 45056;       // keys a CTA holds: 176 KiB next to the histograms (40 KiB)

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
  // neighbouring columns as the two halves of one 64-bit register pair
  __device__ static __forceinline__ void pairs(const uint32_t (&w)[NW], float2 (&f)[NW / 2]) {
#pragma unroll
    for (int i = 0; i < NW / 2; ++i) f[i] = make_float2(__uint_as_float(w[2 * i]), __uint_as_float(w[2 * i + 1]));
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
  // The two bf16 halves of a word become the two halves of one 64-bit value, which the compiler
  // keeps in an aligned register pair: the form the packed fp32x2 multiply-add takes directly.
  __device__ static __forceinline__ void pairs(const uint32_t (&w)[NW], float2 (&f)[NW]) {
#pragma unroll
    for (int i = 0; i < NW; ++i) {
      const unsigned long long pk =
          ((unsigned long long)(w[i] & 0xFFFF0000u) << 32) | (unsigned long long)(w[i] << 16);
      f[i] = make_float2(__uint_as_float((uint32_t)pk), __uint_as_float((uint32_t)(pk >> 32)));
    }
  }
};

struct ScoreTopkParams {
  const void *A_K;      // [N, a_capacity, R]
  const void *q_hat;    // [N, R]
  int64_t a_capacity;
  int64_t candidates;
  int32_t k;
  int32_t seg_len;      // rows per CTA, multiple of kGranule
  uint32_t seg_magic;   // ceil(2^32 / (seg_len / kGranule))
  int32_t *wanted;      // [N, k]
  float *scores_out;    // optional [N, scores_stride]
  int64_t scores_stride;
  int32_t *clear_word;  // optional: set to zero by the kernel
  const uint32_t *keys_in;  // optional [N, keys_stride]: keys already formed by score_keys_kernel
  int64_t keys_stride;
  // optional folded update (fold_update != 0): q_hat is derived from the projection kernel's workspace here,
  // and the last CTA of every cluster applies the head's update while the first runs the hit/miss difference
  int32_t fold_update;
  UpdateArgs upd;
  // optional fused hit/miss difference (table != nullptr): after the selection, the first CTA of
  // every cluster runs slot_diff_head for its head
  int32_t *table;
  uint8_t *mask;
  int32_t *miss_count;
  lrqk_miss *miss_list;
  int32_t *list_len, *diff_status;
};

// Inclusive block scan of NV 32-bit values per thread at once (kThreads threads).  The values are
// replaced by their inclusive prefixes; `tot` receives the block sums.  `scratch`: NV*(kWarps+1) words.
template <int NV>
__device__ __forceinline__ void block_inclusive_scan(uint32_t (&v)[NV], uint32_t *scratch, uint32_t (&tot)[NV]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, v[i], o);
      if (lane >= o) v[i] += x;
    }
  }
  if (lane == 31) {
#pragma unroll
    for (int i = 0; i < NV; ++i) scratch[i * (kWarps + 1) + warp] = v[i];
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const uint32_t w0 = scratch[i * (kWarps + 1) + lane];
      uint32_t w = w0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, w, o);
        if (lane >= o) w += x;
      }
      scratch[i * (kWarps + 1) + lane] = w - w0;  // exclusive warp offsets
      if (lane == 31) scratch[i * (kWarps + 1) + kWarps] = w;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    v[i] += scratch[i * (kWarps + 1) + warp];
    tot[i] = scratch[i * (kWarps + 1) + kWarps];
  }
  __syncthreads();  // scratch may be reused right away
}

// Where the key of local row i lives in shared memory.  Thread t of the compaction owns the
// 4*V consecutive rows [4*V*t, 4*V*(t+1)); its j-th group of four keys is the 16-byte vector
// j*kThreads + t, so that the threads of a warp read neighbouring vectors.  `magic` = ceil(2^32 / V).
__device__ __forceinline__ int key_slot(int i, int V, uint32_t magic) {
  const uint32_t vec = (uint32_t)i >> 2;
  const uint32_t t = V == 1 ? vec : __umulhi(vec, magic);  // vec / V, exact for vec < 2^16 (2^32 / 1 does not fit)
  const uint32_t j = vec - t * (uint32_t)V;
  return (int)(((j * kThreads + t) << 2) | ((uint32_t)i & 3u));
}

// Scores of the rows [seg_begin, seg_begin + seg_rows) of head n, by all kThreads threads of the CTA:
// sink(local_row, score) is called by the lane that ends up with a row's sum, for every local row below the
// returned count (the row count rounded up to whole trips; rows past seg_rows re-read the last row and their
// score is to be discarded).  `qs`: q_hat of the head as fp32 in shared memory, visible to all threads.
template <typename T, int R, typename Sink>
__device__ __forceinline__ int score_rows(const void *A_K, int64_t a_capacity, int n, int64_t seg_begin, int64_t seg_rows,
                                          const float *qs, Sink sink) {
  constexpr int RB = R * (int)sizeof(T);          // bytes per row
  constexpr int VB = RB >= 32 ? 32 : 16;          // bytes per load
  constexpr int VPL = RB >= 64 ? 2 : 1;           // loads per lane and row: a lane covers up to 64 bytes of a row
  constexpr int LPR = RB / (VB * VPL);            // lanes per row
  constexpr int NW = VB / 4;                      // 32-bit words per load
  constexpr int EPV = Unpack<T, NW>::kElts;       // elements per load
  constexpr int EPL = EPV * VPL;                  // elements per lane
  constexpr int RPI = kThreads / LPR;             // rows per CTA-wide load
  constexpr int kUnroll = 4 / VPL;                // rows a thread keeps in flight (128 bytes)
  static_assert(kGranule % (RPI * kUnroll) == 0, "a granule must be a whole number of unrolled loads");
  const int tid = threadIdx.x;
  const int lane_in_row = tid % LPR;
  const int row_in_iter = tid / LPR;
  // q_hat as fp32 pairs in shared memory: every lane of a warp reads the same pair (a broadcast)
  const float4 *q4 = reinterpret_cast<const float4 *>(qs + lane_in_row * EPL);
  const char *base = reinterpret_cast<const char *>(A_K) + ((int64_t)n * a_capacity) * RB + lane_in_row * (VB * VPL);
  const int n_iter_rows = (int)((seg_rows + RPI * kUnroll - 1) / (RPI * kUnroll)) * (RPI * kUnroll);
  // rows past the end of the segment re-read its last row (the result is discarded), so that the
  // loop body is free of special cases
  const int last_row = seg_rows > 0 ? (int)seg_rows - 1 : 0;
  const char *seg_base = seg_rows > 0 ? base + seg_begin * RB : base;  // an empty segment reads (and ignores) row 0

  // Rolling prefetch: a thread keeps kUnroll row pieces in flight; as soon as one has been turned
  // into a key, the piece kUnroll steps ahead is requested into the same registers, so the loads
  // never drain while the dot products are formed.
  Vec<VB> v[kUnroll][VPL];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int local = min(u * RPI + row_in_iter, last_row);
#pragma unroll
    for (int w = 0; w < VPL; ++w) v[u][w].load(seg_base + (int64_t)local * RB + w * VB);
  }
  for (int it = 0; it < n_iter_rows; it += RPI * kUnroll) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int local = it + u * RPI + row_in_iter;
      const int ahead = min(local + RPI * kUnroll, last_row);
      float2 acc2 = make_float2(0.0f, 0.0f);  // even and odd columns of the lane's run
#pragma unroll
      for (int w = 0; w < VPL; ++w) {
        float2 a2[EPV / 2];
        Unpack<T, NW>::pairs(v[u][w].w, a2);
        v[u][w].load(seg_base + (int64_t)ahead * RB + w * VB);
#pragma unroll
        for (int e = 0; e < EPV / 4; ++e) {
          const float4 qq = q4[w * (EPV / 4) + e];
          acc2 = __ffma2_rn(a2[2 * e], make_float2(qq.x, qq.y), acc2);
          acc2 = __ffma2_rn(a2[2 * e + 1], make_float2(qq.z, qq.w), acc2);
        }
      }
      float acc = acc2.x + acc2.y;
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
      if (lane_in_row == 0) sink(local, acc);
    }
  }
  return n_iter_rows;
}

// Work item of the key-streaming kernel: kItemRows rows of one head.
constexpr int kItemRows = 2048;

struct ScoreKeysParams {
  const void *A_K, *q_hat;
  int64_t a_capacity, candidates;
  uint32_t *keys;        // [N, keys_stride]
  int64_t keys_stride;
  float *scores_out;     // optional [N, scores_stride]
  int64_t scores_stride;
  int32_t items_per_head, n_items;
};

// Keys of every candidate row of every head into the workspace.  The items (head, run of kItemRows rows) are
// dealt out in order, an equal share to every CTA, so all SMs stream whatever the head count is.
template <typename T, int R>
__global__ void __launch_bounds__(kThreads, 1) score_keys_kernel(ScoreKeysParams p) {
  __shared__ __align__(16) float qs[R];
  const int tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int first = (int)(((int64_t)blockIdx.x * p.n_items) / gridDim.x);
  const int last = (int)(((int64_t)(blockIdx.x + 1) * p.n_items) / gridDim.x);
  // a CTA's items are consecutive: those of one head form one contiguous run of rows, streamed in one go so
  // that the prefetch pipeline never drains inside it (at most two or three runs per CTA)
  for (int item = first; item < last;) {
    const int n = item / p.items_per_head;
    const int run_end = min(last, (n + 1) * p.items_per_head);
    const int64_t row0 = (int64_t)(item % p.items_per_head) * kItemRows;
    const int64_t rows = min((int64_t)(run_end - item) * kItemRows, p.candidates - row0);
    __syncthreads();  // the previous head's q_hat is no longer read
    if (tid < R) qs[tid] = Elt<T>::to_float(reinterpret_cast<const T *>(p.q_hat)[(int64_t)n * R + tid]);
    __syncthreads();
    uint32_t *kout = p.keys + (int64_t)n * p.keys_stride + row0;
    score_rows<T, R>(p.A_K, p.a_capacity, n, row0, rows, qs, [&](int local, float acc) {
      if (local < rows) {
        kout[local] = order_key(acc);
        if (p.scores_out) p.scores_out[(int64_t)n * p.scores_stride + row0 + local] = acc;
      }
    });
    item = run_end;
  }
}

template <typename T, int R>
__global__ void __launch_bounds__(kThreads, 1) score_topk_kernel(ScoreTopkParams p) {
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int csize = (int)cluster.num_blocks();
  const int n = blockIdx.y;
  const int tid = threadIdx.x;

  extern __shared__ __align__(16) uint32_t smem[];
  uint32_t *keys = smem;                       // [seg_len]
  uint32_t *hist = keys + p.seg_len;           // [3][kBins] this CTA's own histogram of each pass
  uint32_t *sums = hist + 3 * kBins;           // [tot, low][kBins] cluster-wide histograms of passes 0 and 2, filled by the peers
  uint32_t *scratch = sums + 2 * kBins;          // [2*(kWarps + 1)]
  uint32_t *bcast = scratch + 2 * (kWarps + 1);  // [3 passes][4] (+2: keeps what follows on a 16-byte boundary)
  float *qs = reinterpret_cast<float *>(bcast + 14);  // [R] q_hat in fp32, read as float4

  pdl_launch_dependents();
  for (int i = tid; i < 5 * kBins; i += kThreads) hist[i] = 0;
  // no peer may add to this CTA's cluster-wide histograms before they are cleared
  cluster.sync();
  pdl_wait();  // everything above touched shared memory only
  if (p.clear_word && n == 0 && rank == 0 && tid == 0) *p.clear_word = 0;
  const int V = p.seg_len / (4 * kThreads);  // 16-byte key vectors per thread
  const uint32_t magic = p.seg_magic;

  // ---- streaming pass: scores -> keys in shared memory, pass-0 histogram on the fly -------
  const int64_t seg_begin = (int64_t)rank * p.seg_len;
  int64_t seg_rows = p.candidates - seg_begin;   // rows of this segment that hold candidates
  if (seg_rows < 0) seg_rows = 0;
  if (seg_rows > p.seg_len) seg_rows = p.seg_len;
  int n_iter_rows;
  int chosen = 0;
  if (p.keys_in != nullptr) {
    // the keys were formed by score_keys_kernel: fetch this segment's (they sit in L2), four per thread and trip
    const uint32_t *kin = p.keys_in + (int64_t)n * p.keys_stride + seg_begin;
    n_iter_rows = (int)((seg_rows + 4 * kThreads - 1) / (4 * kThreads)) * (4 * kThreads);
    for (int i0 = 4 * tid; i0 < n_iter_rows; i0 += 4 * kThreads) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (i0 + 3 < seg_rows) {
        v = __ldcg(reinterpret_cast<const uint4 *>(kin + i0));
      } else {
        if (i0 < seg_rows) v.x = __ldcg(kin + i0);
        if (i0 + 1 < seg_rows) v.y = __ldcg(kin + i0 + 1);
        if (i0 + 2 < seg_rows) v.z = __ldcg(kin + i0 + 2);
      }
      const uint32_t kk[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (i0 + c < seg_rows) atomicAdd(&hist[kk[c] >> 21], 1u);
        keys[key_slot(i0 + c, V, magic)] = i0 + c < seg_rows ? kk[c] : 0u;
      }
    }
  } else {
    if (p.fold_update) {
      // the reference's early-exit decision over all heads, then this head's projected query of that
      // alternation, rounded to the storage dtype as the stored q_hat is
      chosen = update_chosen<R>(p.upd, reinterpret_cast<float *>(scratch));
      const float *w = p.upd.ws + ((int64_t)n * p.upd.max_iter + chosen) * (2 * R + 2);
      if (tid < R) qs[tid] = Elt<T>::to_float(Elt<T>::from_float(w[tid]));
      if (n == 0 && rank == 0 && tid == 0 && p.upd.iters_out) *p.upd.iters_out = chosen + 1;
    } else if (tid < R) {
      qs[tid] = Elt<T>::to_float(reinterpret_cast<const T *>(p.q_hat)[(int64_t)n * R + tid]);
    }
    __syncthreads();
    n_iter_rows = score_rows<T, R>(p.A_K, p.a_capacity, n, seg_begin, seg_rows, qs, [&](int local, float acc) {
      uint32_t key = 0;
      if (local < seg_rows) {
        key = order_key(acc);
        atomicAdd(&hist[key >> 21], 1u);
        if (p.scores_out) p.scores_out[(int64_t)n * p.scores_stride + seg_begin + local] = acc;
      }
      keys[key_slot(local, V, magic)] = key;
    });
  }
  for (int i = n_iter_rows + tid; i < p.seg_len; i += kThreads) keys[key_slot(i, V, magic)] = 0;  // padding sorts last
  __syncthreads();

  // ---- radix select of the k-th largest key over the whole cluster ---------------------------
  // Three passes (11 + 11 + 10 bits).  A pass: local histogram of the digit among the keys that
  // match the prefix found so far; one cluster barrier; every CTA reads all histograms of the
  // cluster (two bins per thread and peer) and picks the digit itself.  From the same reads it
  // learns how many keys above the chosen digit lie in lower-ranked CTAs.
  uint32_t prefix = 0;
  uint32_t need = (uint32_t)p.k;
  uint32_t out_base = 0;  // selected keys held by lower-ranked CTAs
  uint32_t quota = 0;     // how many keys equal to the threshold this CTA contributes
  unsigned long long sel = 0ull, und = 0ull;  // this thread's keys: surely selected / still undecided (bit = position in its run)
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int bits = pass == 2 ? 10 : 11;
    const uint32_t dmask = (1u << bits) - 1;
    uint32_t *hl = hist + pass * kBins;
    if (pass == 1) {
      // The only pass over all keys after the stream: every thread sorts the keys of its own run
      // into "above the chosen digit" (sel) and "equal to it" (und: undecided), one bit per key,
      // and histograms the next digit of the undecided ones.  Later passes only walk those bits.
      const uint4 *k4 = reinterpret_cast<const uint4 *>(keys);
      for (int j = 0; j < V; ++j) {
        const uint4 v = k4[j * kThreads + tid];
        const uint32_t kk[4] = {v.x, v.y, v.z, v.w};
        uint32_t above = 0u, equal = 0u;  // one bit per key of this group of four
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t top = kk[c] >> 21;
          above |= (uint32_t)(top > prefix) << c;
          if (top == prefix) {
            equal |= 1u << c;
            atomicAdd(&hl[(kk[c] >> 10) & dmask], 1u);
          }
        }
        sel |= (unsigned long long)above << (4 * j);
        und |= (unsigned long long)equal << (4 * j);
      }
      __syncthreads();
    } else if (pass == 2) {
      unsigned long long m = und;
      while (m) {
        const int i = __ffsll((long long)m) - 1;
        m &= m - 1;
        const uint32_t key = keys[(((i >> 2) * kThreads + tid) << 2) | (i & 3)];
        const uint32_t digit = (key >> 10) & 0x7FFu;
        const uint32_t chosen = prefix & 0x7FFu;  // the digit pass 1 settled on
        if (digit != chosen) und &= ~(1ull << i);
        if (digit > chosen) sel |= 1ull << i;
        if (digit == chosen) atomicAdd(&hl[key & dmask], 1u);
      }
      __syncthreads();
    }
    // Every CTA ADDS its histogram to the cluster-wide one held by each CTA of the cluster (remote
    // shared-memory atomics on integers: the sums do not depend on the order), and to the "held by
    // lower-ranked CTAs" histogram of the CTAs ranked above it.  After the barrier everything a CTA needs
    // is in its own shared memory; nobody reads a peer's memory.  Two sets alternate; the set of pass 0
    // is cleared again once it has been read, for pass 2.
    // Passes 0 and 2 (a few dozen occupied bins): every CTA ADDS its histogram to the cluster-wide one held
    // by each CTA of the cluster (remote shared-memory atomics on integers: the sums do not depend on the
    // order), and to the "held by lower-ranked CTAs" histogram of the CTAs ranked above it; after the barrier
    // everything a CTA needs is in its own shared memory.  Pass 1 (nearly every bin occupied) reads the peers'
    // histograms after the barrier instead: two bins per thread and peer cost less than that many atomics.
    uint32_t *tot_s = sums, *low_s = sums + kBins;
    uint32_t tot[2] = {0u, 0u}, low[2] = {0u, 0u};
    if (pass != 1) {
      const uint2 own = *reinterpret_cast<const uint2 *>(hl + 2 * tid);
      if (own.x | own.y) {
        for (int c = 0; c < csize; ++c) {
          uint32_t *rt = c == rank ? tot_s : cluster.map_shared_rank(tot_s, c);
          if (own.x) atomicAdd(rt + 2 * tid, own.x);
          if (own.y) atomicAdd(rt + 2 * tid + 1, own.y);
          if (c > rank) {
            uint32_t *rl = cluster.map_shared_rank(low_s, c);
            if (own.x) atomicAdd(rl + 2 * tid, own.x);
            if (own.y) atomicAdd(rl + 2 * tid + 1, own.y);
          }
        }
      }
    }
    cluster.sync();  // every CTA's histogram of this pass is complete, its additions have arrived
    if (pass != 1) {
      const uint2 tv = *reinterpret_cast<const uint2 *>(tot_s + 2 * tid);
      const uint2 lv = *reinterpret_cast<const uint2 *>(low_s + 2 * tid);
      tot[0] = tv.x; tot[1] = tv.y; low[0] = lv.x; low[1] = lv.y;
      if (pass == 0) {  // pass 2 uses the same arrays: clear them (the peers add to them only after the next barrier)
        *reinterpret_cast<uint2 *>(tot_s + 2 * tid) = make_uint2(0u, 0u);
        *reinterpret_cast<uint2 *>(low_s + 2 * tid) = make_uint2(0u, 0u);
      }
    } else {
      for (int c = 0; c < csize; ++c) {
        const uint2 v = *reinterpret_cast<const uint2 *>(cluster.map_shared_rank(hl, c) + 2 * tid);
        tot[0] += v.x; tot[1] += v.y;
        if (c < rank) { low[0] += v.x; low[1] += v.y; }
      }
    }
    // keys in the bins ABOVE this thread's two bins, and those of them held by lower-ranked CTAs: a scan by
    // shuffles inside the warp, the warp totals through shared memory
    const uint32_t mine = tot[0] + tot[1], mine_low = low[0] + low[1];
    uint32_t inc = mine, inc_low = mine_low;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o), y = __shfl_up_sync(0xFFFFFFFFu, inc_low, o);
      if ((tid & 31) >= o) { inc += x; inc_low += y; }
    }
    const uint32_t warp_tot = __shfl_sync(0xFFFFFFFFu, inc, 31), warp_tot_low = __shfl_sync(0xFFFFFFFFu, inc_low, 31);
    if ((tid & 31) == 0) { scratch[tid >> 5] = warp_tot; scratch[kWarps + (tid >> 5)] = warp_tot_low; }
    __syncthreads();
    uint32_t above, above_low;
    {
      // totals of the warps above this one: lane l holds warp l's totals, masked and summed
      const int lane = tid & 31, wp = tid >> 5;
      uint32_t a = lane > wp ? scratch[lane] : 0u, al = lane > wp ? scratch[kWarps + lane] : 0u;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xFFFFFFFFu, a, o); al += __shfl_xor_sync(0xFFFFFFFFu, al, o); }
      above = a + (warp_tot - inc);
      above_low = al + (warp_tot_low - inc_low);
    }
    uint32_t *bc = bcast + 4 * pass;
    if (above < need && need <= above + mine) {
#pragma unroll
      for (int j = 1; j >= 0; --j) {
        if (above + tot[j] >= need) {
          bc[0] = (uint32_t)(2 * tid + j);
          bc[1] = need - above;
          bc[2] = above_low;
          bc[3] = low[j];
          break;
        }
        above += tot[j];
        above_low += low[j];
      }
    }
    __syncthreads();
    prefix = (prefix << bits) | bc[0];
    need = bc[1];
    out_base += bc[2];
    if (pass == 2) {
      const uint32_t ties_low = bc[3];          // keys equal to the threshold in lower-ranked CTAs
      const uint32_t ties_mine = hl[bc[0]];
      const uint32_t left = need > ties_low ? need - ties_low : 0u;
      quota = ties_mine < left ? ties_mine : left;
      out_base += ties_low < need ? ties_low : need;
    }
  }
  const uint32_t T_key = prefix;  // the k-th largest key
  // the CTA that will run the hit/miss difference asks for its slot-table entries now: they do not depend on
  // the selection, and the load has returned by the time the compaction and the cluster barrier are through
  DiffPre tab_pre = DiffPre{0, 0, 0, 0, false};
  if (p.table != nullptr && rank == 0 && p.k <= kDiffPre * kDThreads) tab_pre = slot_diff_preload(n, p.table, p.k);

  // ---- ordered compaction: every thread owns 4*V consecutive rows -----------------------------
  // The undecided keys (a handful per cluster by now) are settled against the threshold; the
  // selected keys of a thread are then the set bits of two masks.  Counts travel as one word:
  // keys above the threshold in the low half, equal keys in the high half.
  unsigned long long tie = 0ull;
  {
    unsigned long long m = und;
    while (m) {
      const int i = __ffsll((long long)m) - 1;
      m &= m - 1;
      const uint32_t key = keys[(((i >> 2) * kThreads + tid) << 2) | (i & 3)];
      if (key > T_key) sel |= 1ull << i;
      if (key == T_key) tie |= 1ull << i;
    }
  }
  const uint32_t own = (uint32_t)__popcll(sel) | ((uint32_t)__popcll(tie) << 16);
  uint32_t cnt[1] = {own}, cta_total[1];
  block_inclusive_scan<1>(cnt, scratch, cta_total);
  if (own != 0u) {
    const uint32_t at = cnt[0] - own;
    uint32_t g_at = at & 0xFFFFu, e_at = at >> 16;
    int32_t *out = p.wanted + (int64_t)n * p.k;
    const int32_t first = (int32_t)seg_begin + tid * 4 * V;
    unsigned long long m = sel | tie;
    while (m) {  // ascending bit = ascending position
      const int i = __ffsll((long long)m) - 1;
      m &= m - 1;
      const bool is_e = (tie >> i) & 1ull;
      if (!is_e || e_at < quota) {
        const uint32_t pos = out_base + g_at + (e_at < quota ? e_at : quota);
        if (pos < (uint32_t)p.k) out[pos] = first + i;
      }
      g_at += is_e ? 0u : 1u;
      e_at += is_e ? 1u : 0u;
    }
  }
  if (p.table != nullptr) {
    // fused hit/miss difference: once every CTA of the cluster has written its part of `wanted`
    // (release/acquire through the cluster barrier), the first CTA diffs the head's wanted set
    // against the slot table; the keys' shared memory is free by now
    __threadfence();
    cluster.sync();
    if (rank == 0)
      slot_diff_head(n, p.table, p.wanted, p.mask, p.miss_count, p.miss_list, p.list_len, p.diff_status, p.k,
                     reinterpret_cast<unsigned char *>(smem), tab_pre);
  }
  if (p.fold_update && rank == csize - 1) {
    // the head's update of B_Q, B_K, q_hat and the new A_K row: by the cluster's last CTA, which is idle
    // while the first runs the difference (a cluster of one does it afterwards); the keys' memory is free
    __syncthreads();
    update_head<T, R>(p.upd, n, chosen, reinterpret_cast<float *>(smem));
  }
}

// Shared memory of the select kernel for a segment of seg_len keys (and, fused with the hit/miss difference, at
// least what that needs).
static size_t score_smem_bytes(int seg_len, int r, int k_for_diff, int d_for_update = 0) {
  size_t smem = ((size_t)seg_len + 5 * kBins + 2 * (kWarps + 1) + 14 + r) * sizeof(uint32_t);
  if (k_for_diff > 0 && slot_diff_smem_bytes(k_for_diff) > smem) smem = slot_diff_smem_bytes(k_for_diff);
  const size_t upd = d_for_update > 0 ? sizeof(float) * (size_t)update_head_smem_floats(r, d_for_update) : 0;
  return smem > upd ? smem : upd;
}

template <typename T, int R>
int launch_score_topk(const ScoreTopkParams &p, int n_heads, int csize, cudaStream_t stream) {
  static_assert((5 * kBins + 2 * (kWarps + 1) + 14) % 4 == 0, "q_hat must start on a 16-byte boundary");
  const size_t smem = score_smem_bytes(p.seg_len, R, p.table != nullptr ? p.k : 0, p.fold_update ? p.upd.head_dim : 0);
  auto kern = score_topk_kernel<T, R>;
  static SmemOptIn opt_in;
  LRQK_CUDA_TRY(opt_in.ensure(kern, smem));
  if (csize > 8)   // clusters of 16 need the non-portable opt-in (per device, cheap: only the very long contexts get here)
    LRQK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  LRQK_CUDA_TRY(launch_dependent(kern, dim3(csize, n_heads, 1), dim3(kThreads), smem, stream, csize, p));
  return LRQK_OK;
}

template <typename T, int R>
int launch_score_keys(const ScoreKeysParams &p, cudaStream_t stream) {
  const int grid = p.n_items < kNumSMs ? p.n_items : kNumSMs;
  LRQK_CUDA_TRY(launch_dependent(score_keys_kernel<T, R>, dim3(grid), dim3(kThreads), 0, stream, 0, p));
  return LRQK_OK;
}

template <typename T>
int dispatch_keys(int r, const ScoreKeysParams &p, cudaStream_t stream) {
  switch (r) {
    case 8: return launch_score_keys<T, 8>(p, stream);
    case 16: return launch_score_keys<T, 16>(p, stream);
    case 32: return launch_score_keys<T, 32>(p, stream);
    case 64: return launch_score_keys<T, 64>(p, stream);
    default: return LRQK_EUNSUPPORTED;
  }
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

// How many clusters of `cs` CTAs of the select kernel the current device keeps resident at once (one CTA per SM;
// a cluster must fit inside one GPC, so it is not simply SMs / cs).  Asked of the runtime once per (kernel,
// cluster size, device); 0 when it cannot be told.
template <typename T, int R>
int resident_clusters_of(int cs, size_t smem) {
  static std::mutex mu;
  static int cache[kMaxDevices][9];  // 0 = not asked yet, -1 = unknown
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || cs < 1 || cs > 8) { cudaGetLastError(); return 0; }
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev][cs] == 0) {
    auto kern = score_topk_kernel<T, R>;
    int n = 0;
    // the largest shared-memory size any plan uses, so that the answer holds for every segment length
    const size_t smem_max = score_smem_bytes(kMaxSeg, R, 0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cs, 1, 1);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_max;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) { cudaGetLastError(); n = -1; }
    cache[dev][cs] = n > 0 ? n : -1;
  }
  (void)smem;
  return cache[dev][cs] > 0 ? cache[dev][cs] : 0;
}

static int resident_clusters(const lrqk_layer *L, int cs, size_t smem) {
  int n = 0;
#define LRQK_RC(T, R) n = resident_clusters_of<T, R>(cs, smem)
  if (L->dtype == LRQK_BF16) {
    switch (L->r) { case 8: LRQK_RC(__nv_bfloat16, 8); break; case 16: LRQK_RC(__nv_bfloat16, 16); break;
                    case 32: LRQK_RC(__nv_bfloat16, 32); break; case 64: LRQK_RC(__nv_bfloat16, 64); break; default: break; }
  } else {
    switch (L->r) { case 8: LRQK_RC(float, 8); break; case 16: LRQK_RC(float, 16); break;
                    case 32: LRQK_RC(float, 32); break; case 64: LRQK_RC(float, 64); break; default: break; }
  }
#undef LRQK_RC
  if (n <= 0) n = cs >= 7 ? 15 : (cs >= 5 ? 24 : (cs == 4 ? 36 : kNumSMs / cs));  // estimate for a 148-SM part
  return n;
}

// Cluster size (1..8, any value) and segment length for `candidates` rows per head and n_heads heads.
// One CTA per SM (its keys fill most of the SM's shared memory).  Every cluster size whose segment fits is
// rated by the time it implies: waves of resident clusters times (rows a CTA streams + the fixed cost of the
// select passes, expressed in rows); the cheapest wins, the smaller cluster on a draw.
int plan_score_topk(const lrqk_layer *L, int64_t candidates, int n_heads, int *csize_out, int *seg_len_out) {
  const int64_t select_cost_rows = 10240;  // ~12 us of select passes at the ~52 GB/s one SM streams (64-byte rows)
  int best = -1;
  int64_t best_cost = 0;
  for (int cs = 1; cs <= 8; ++cs) {
    const int64_t seg = ceil_div64(ceil_div64(candidates, cs), kGranule) * kGranule;
    if (seg > kMaxSeg) continue;
    if (cs > 1 && ceil_div64(candidates, cs) < kGranule && best >= 0) break;  // a CTA keeps at least one granule
    const int resident = resident_clusters(L, cs, 0);
    const int64_t waves = ceil_div64(n_heads, resident > 0 ? resident : 1);
    const int64_t cost = waves * (seg + select_cost_rows);
    if (best < 0 || cost < best_cost) { best = cs; best_cost = cost; }
  }
  if (best < 0) {  // longer than eight segments: a non-portable cluster of 16
    const int64_t seg = ceil_div64(ceil_div64(candidates, 16), kGranule) * kGranule;
    if (seg > kMaxSeg) return LRQK_EUNSUPPORTED;
    best = 16;
  }
  *csize_out = best;
  *seg_len_out = (int)(ceil_div64(ceil_div64(candidates, best), kGranule) * kGranule);
  return LRQK_OK;
}

// Whether the keys should be formed by the all-SM streaming kernel first: only when the clusters of the
// one-kernel plan would occupy less than an eighth of the SMs.  (Measured at 131072 rows: from 4 heads on --
// 32 CTAs -- one kernel is as quick or quicker, because the select passes, not the stream, set its time; and
// only the one-kernel plan can apply the projection's update in the same launch.)
static bool plan_wants_key_pass(int n_heads, int csize) { return n_heads * csize * 8 < kNumSMs; }

static int64_t keys_stride_for(int64_t rows) { return (rows + 3) / 4 * 4; }

}  // namespace lrqk

bool lrqk::score_topk_can_fold_update(const lrqk_layer *L, int64_t candidates, void *workspace, size_t workspace_bytes) {
  if (!L || check_layer(L) != LRQK_OK || candidates <= L->k || L->head_dim > 128) return false;
  const int n_heads = L->bsz * L->q_heads;
  int csize = 1, seg_len = 0;
  if (plan_score_topk(L, candidates, n_heads, &csize, &seg_len) != LRQK_OK) return false;
  const bool key_pass = workspace && plan_wants_key_pass(n_heads, csize) &&
                        workspace_bytes >= sizeof(uint32_t) * (size_t)n_heads * (size_t)keys_stride_for(candidates);
  return !key_pass;
}

extern "C" size_t lrqk_score_topk_workspace_bytes(const lrqk_layer *L, int64_t max_candidates) {
  if (!L || max_candidates <= 0 || lrqk::check_layer(L) != LRQK_OK) return 0;
  const int n_heads = L->bsz * L->q_heads;
  // the cluster size only grows with the candidate count, so the smallest count decides whether any call
  // may take the two-kernel plan
  int csize = 1, seg_len = 0;
  if (lrqk::plan_score_topk(L, L->k + 1, n_heads, &csize, &seg_len) != LRQK_OK) return 0;
  if (!lrqk::plan_wants_key_pass(n_heads, csize)) {
    if (lrqk::plan_score_topk(L, max_candidates, n_heads, &csize, &seg_len) != LRQK_OK) return 0;
    if (!lrqk::plan_wants_key_pass(n_heads, csize)) return 0;
  }
  return sizeof(uint32_t) * (size_t)n_heads * (size_t)lrqk::keys_stride_for(max_candidates);
}

extern "C" int lrqk_score_topk(const lrqk_layer *L, const void *q_hat, int64_t candidates, int32_t *wanted,
                               float *scores_out, int64_t scores_stride, void *workspace, size_t workspace_bytes,
                               lrqk_stream_t stream) {
  return lrqk::score_topk_enqueue(L, q_hat, candidates, wanted, scores_out, scores_stride, nullptr,
                                  lrqk::as_stream(stream), nullptr, workspace, workspace_bytes);
}

int lrqk::score_topk_enqueue(const lrqk_layer *L, const void *q_hat, int64_t candidates, int32_t *wanted,
                             float *scores_out, int64_t scores_stride, int32_t *clear_word, cudaStream_t stream,
                             const FusedDiff *diff, void *workspace, size_t workspace_bytes, const UpdateArgs *update) {
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
  p.clear_word = clear_word;
  p.keys_in = nullptr; p.keys_stride = 0;
  p.fold_update = 0;
  p.table = nullptr; p.mask = nullptr; p.miss_count = nullptr; p.miss_list = nullptr; p.list_len = nullptr; p.diff_status = nullptr;
  if (diff) {
    if (!L->table || !diff->mask || !diff->miss_count || !diff->list || !diff->list_len || !diff->status) return LRQK_EINVAL;
    if (slot_diff_smem_bytes(L->k) > 200 * 1024) return LRQK_EUNSUPPORTED;
    p.table = L->table; p.mask = diff->mask; p.miss_count = diff->miss_count; p.miss_list = diff->list;
    p.list_len = diff->list_len; p.diff_status = diff->status;
  }
  int csize = 1, seg_len = 0;
  rc = plan_score_topk(L, candidates, n_heads, &csize, &seg_len);
  if (rc != LRQK_OK) return rc;
  p.seg_len = seg_len;
  {
    const uint32_t v = (uint32_t)(seg_len / kGranule);
    p.seg_magic = (uint32_t)((0x100000000ull + v - 1) / v);
  }
  const int64_t kstride = keys_stride_for(candidates);
  const bool key_pass = workspace && plan_wants_key_pass(n_heads, csize) &&
                        workspace_bytes >= sizeof(uint32_t) * (size_t)n_heads * (size_t)kstride;
  if (update) {
    if (key_pass || L->head_dim > 128) return LRQK_EINVAL;  // callers ask score_topk_can_fold_update() first
    p.fold_update = 1;
    p.upd = *update;
  }
  if (key_pass) {
    // few heads: form the keys on all SMs first, the clusters then select from the workspace
    ScoreKeysParams kp;
    kp.A_K = L->A_K; kp.q_hat = q_hat; kp.a_capacity = L->a_capacity; kp.candidates = candidates;
    kp.keys = reinterpret_cast<uint32_t *>(workspace); kp.keys_stride = kstride;
    kp.scores_out = scores_out; kp.scores_stride = scores_stride;
    kp.items_per_head = (int32_t)ceil_div64(candidates, kItemRows);
    kp.n_items = kp.items_per_head * n_heads;
    LRQK_DISPATCH_DTYPE(L->dtype, T, rc = dispatch_keys<T>(L->r, kp, stream));
    if (rc != LRQK_OK) return rc;
    p.keys_in = kp.keys; p.keys_stride = kstride;
    p.scores_out = nullptr;
  }
  LRQK_DISPATCH_DTYPE(L->dtype, T, return dispatch_rank<T>(L->r, p, n_heads, csize, stream));
  return LRQK_EUNSUPPORTED;
}
